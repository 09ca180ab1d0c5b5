"""Trainer / callbacks / metrics / CLI entry points on CPU (tiny 2-layer model, synthetic tokens)."""
import json
import os
import subprocess
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

MODEL = dict(arch=dict(type="LlamaForCausalLM"),
             model_config=dict(model_type="llama", vocab_size=128, hidden_size=64, intermediate_size=128, num_hidden_layers=2,
                               num_attention_heads=4, num_key_value_heads=2, seq_length=32, max_position_embeddings=32,
                               params_dtype="float32", compute_dtype="float32"))


def _cfg(out, **over):
    cfg = dict(output_dir=str(out), run_mode="train", use_legacy=False, seed=3, model=MODEL,
               runner_config=dict(epochs=1, batch_size=2),
               train_dataset=dict(data_loader=dict(type="MockDataLoader", num_samples=16, seq_length=32, vocab_size=128, seed=5)),
               train_dataset_task=dict(type="CausalLanguageModelDataset"),
               optimizer=dict(type="AdamW", learning_rate=1e-3, betas=[0.9, 0.95]),
               lr_schedule=dict(type="ConstantWarmUpLR", learning_rate=1e-3, warmup_steps=0, total_steps=-1),
               context=dict(device_target="CPU"),
               callbacks=[dict(type="MFLossMonitor"), dict(type="CheckpointMonitor", save_checkpoint_steps=4, prefix="t")])
    cfg.update(over)
    return cfg


def _fresh():
    from mindformers_b200.core import context
    context._CONTEXT = None


def test_train_saves_and_resume_reproduces_losses(tmp_path):
    from mindformers_b200.trainer import Trainer
    _fresh()
    full = Trainer(args=_cfg(tmp_path / "a"))
    full.train()
    ref = full.trainer.loss_history
    assert len(ref) == 8
    ck = tmp_path / "a" / "checkpoint"
    assert sorted(os.listdir(ck / "rank_0")) == ["meta.json", "t_rank_0-1_4.safetensors", "t_rank_0-1_8.safetensors"]
    assert json.load(open(ck / "rank_0" / "meta.json"))["last_step"] == 8
    # drop the final checkpoint so that the resume point is step 4, then continue: losses 5..8 must match
    os.remove(ck / "rank_0" / "t_rank_0-1_8.safetensors")
    json.dump({"last_epoch": 1, "last_step": 4, "last_ckpt_file": "t_rank_0-1_4.safetensors"}, open(ck / "rank_0" / "meta.json", "w"))
    _fresh()
    again = Trainer(args=_cfg(tmp_path / "b", load_checkpoint=str(ck), resume_training=True))
    again.train()
    got = again.trainer.loss_history
    assert len(got) == 4
    for a, b in zip(ref[4:], got):
        assert abs(a - b) < 5e-3, (ref, got)


def test_training_arguments_roundtrip_and_monitors(tmp_path):
    from mindformers_b200.core.callback import GracefulExitCallback, TrainingStateMonitor
    from mindformers_b200.trainer import Trainer, TrainingArguments
    args = TrainingArguments(output_dir=str(tmp_path), num_train_epochs=1, batch_size=2, learning_rate=2e-3, lr_scheduler_type="linear",
                             warmup_steps=1, save_strategy="no", use_cpu=True)
    cfg = args.convert_args_to_mindformers_config()
    assert cfg["lr_schedule"]["type"] == "LinearWithWarmUpLR" and cfg["optimizer"]["learning_rate"] == 2e-3
    assert cfg["context"]["device_target"] == "CPU"
    flag = tmp_path / "graceful_exit.json"
    json.dump({"GracefulExit": 1}, open(flag, "w"))
    _fresh()
    c = _cfg(tmp_path / "g", callbacks=[dict(type="MFLossMonitor")])
    t = Trainer(args=c, callbacks=None)
    cbs = t.trainer.create_callbacks(t.config, {}) + [GracefulExitCallback(str(flag)),
                                                      TrainingStateMonitor(config=dict(weight_state_format=["log"], target=["final_layernorm"]))]
    t.callbacks = cbs
    st = t.train()
    assert st.global_step == 1 and st.stop_reason == "graceful_exit"
    assert any(k.startswith("weight_norm/") for k in cbs[-1].stats[0])


def test_spike_and_nan_detection():
    from mindformers_b200.core.callback import RunContext, TrainingStateMonitor
    import tempfile
    d = tempfile.mkdtemp()
    mon = TrainingStateMonitor(config=dict(global_norm_spike_threshold=2.0, check_for_global_norm=True,
                                           global_norm_record_path=os.path.join(d, "spike.json")))
    ctx = RunContext(global_step=7, loss=1.0, global_norm=5.0)
    with pytest.raises(RuntimeError, match="TREError"):
        mon.on_step_end(ctx)
    assert "7" in json.load(open(os.path.join(d, "spike.json")))
    with pytest.raises(RuntimeError, match="loss is nan"):
        mon.on_step_end(RunContext(global_step=8, loss=float("nan"), global_norm=1.0))


def test_metrics():
    from mindformers_b200.core.metric import ADGENMetric, EmF1Metric, EntityScore, PerplexityMetric, PromptAccMetric
    torch.manual_seed(0)
    logits, labels = torch.randn(2, 6, 11), torch.randint(0, 11, (2, 6))
    m = PerplexityMetric()
    m.update(logits, labels, torch.ones(2, 6))
    want = torch.nn.functional.cross_entropy(logits[:, :-1].reshape(-1, 11), labels[:, 1:].reshape(-1))
    assert abs(m.eval()["loss"] - float(want)) < 1e-5
    em = EmF1Metric()
    em.update(["The cat sat."], ["cat sat"])
    assert em.eval()["Em"] == 100.0
    ad = ADGENMetric()
    ad.update(["abcd"], ["abcd"])
    assert ad.eval()["rouge-l"] == pytest.approx(100.0)
    es = EntityScore(["O", "B-P", "I-P"])
    es.update([[0, 1, 2, 0]], [[0, 1, 2, 0]])
    assert es.eval()["f1"] == 1.0
    pa = PromptAccMetric()
    lg = torch.full((2, 3, 5), -5.0)
    ids = torch.tensor([[0, 1, 2], [0, 3, 4]])
    lg[0, 0, 1] = lg[0, 1, 2] = 5.0      # candidate 0 is the likely continuation
    pa.update(lg, ids, torch.ones(2, 3), torch.tensor([0]))
    assert pa.eval()["Acc"] == 1.0


def test_cli_train_eval_predict(tmp_path):
    env = dict(os.environ, PYTHONPATH=ROOT)
    base = [sys.executable, os.path.join(ROOT, "run_mindformer.py"), "--config", os.path.join(ROOT, "configs/general/run_general_task.yaml"),
            "--output_dir", str(tmp_path), "--context.device_target", "CPU"]
    r = subprocess.run(base + ["--runner_config.stop_step=2"], capture_output=True, text=True, env=env, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    assert "step:[    2/" in r.stderr + r.stdout
    ck = os.path.join(str(tmp_path), "checkpoint")
    r = subprocess.run(base + ["--run_mode", "predict", "--load_checkpoint", ck, "--predict_data", "hello", "--use_parallel", "False"],
                       capture_output=True, text=True, env=env, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    assert os.path.exists(os.path.join(str(tmp_path), "text_generation_result.txt"))


def test_convert_weight_roundtrip(tmp_path):
    from safetensors.torch import load_file
    from mindformers_b200.models import LlamaConfig, LlamaForCausalLM
    import convert_weight
    cfg = LlamaConfig(vocab_size=64, hidden_size=32, intermediate_size=64, num_hidden_layers=1, num_attention_heads=4,
                      num_key_value_heads=2, params_dtype="float32", compute_dtype="float32")
    torch.manual_seed(0)
    m = LlamaForCausalLM(cfg, device="cpu")
    m.save_pretrained(str(tmp_path / "hf"), hf_names=True)
    out = convert_weight.main(["--model", "llama", "--input_path", str(tmp_path / "hf"), "--output_path", str(tmp_path / "mf")])
    sd = load_file(out)
    own = dict(m.model.named_parameters())
    assert set(own) <= set(sd)
    for k, v in own.items():
        assert torch.equal(sd[k], v.detach()), k
    back = convert_weight.main(["--model", "llama", "--reversed", "--input_path", out, "--output_path", str(tmp_path / "hf2"),
                                "--config", str(tmp_path / "hf" / "config.json")])
    a, b = load_file(back), {}
    for f in os.listdir(tmp_path / "hf"):
        if f.endswith(".safetensors"):
            b.update(load_file(str(tmp_path / "hf" / f)))
    assert set(a) == set(b) and all(torch.equal(a[k], b[k]) for k in a)
    # the same conversion with the paths taken from a convert_config YAML
    import yaml
    yml = tmp_path / "run_convert.yaml"
    yaml.safe_dump({"llama": {"input_path": str(tmp_path / "hf"), "output_path": str(tmp_path / "mf2"), "dtype": None}},
                   open(yml, "w"))
    out2 = convert_weight.main(["--model", "llama", "--convert_config", str(yml)])
    assert all(torch.equal(load_file(out2)[k], sd[k]) for k in sd)
    shipped = yaml.safe_load(open(os.path.join(ROOT, "configs", "convert_config", "run_convert.yaml")))
    assert set(shipped) >= {"llama", "qwen3_moe", "deepseekv3"} and set(shipped) <= set(convert_weight.convert_map)


def test_config_arguments_sections():
    from mindformers_b200.trainer import (CheckpointConfig, ConfigArguments, LRConfig, OptimizerConfig, ParallelConfig,
                                          RunnerConfig, Trainer)
    import pytest as _pytest
    args = ConfigArguments(
        output_dir="./out_cfg", seed=7, runner_config=RunnerConfig(epochs=2, batch_size=4),
        optimizer=OptimizerConfig(optim_type="AdamW", learning_rate=3e-4, weight_decay=0.05),
        lr_schedule=LRConfig(lr_type="CosineWithWarmUpLR", warmup_steps=10),
        parallel_config=ParallelConfig(data_parallel=1, model_parallel=1),
        save_checkpoint=CheckpointConfig(save_checkpoint_steps=50, keep_checkpoint_max=2))
    cfg = args.to_config()
    assert cfg["runner_config"] == {"epochs": 2, "batch_size": 4}
    assert cfg["optimizer"]["type"] == "AdamW" and cfg["optimizer"]["learning_rate"] == 3e-4
    assert cfg["lr_schedule"] == {"type": "CosineWithWarmUpLR", "warmup_steps": 10}
    assert cfg["callbacks"][-1]["type"] == "CheckpointMonitor" and cfg["callbacks"][-1]["save_checkpoint_steps"] == 50
    assert "save_checkpoint" not in cfg
    with _pytest.raises(KeyError):
        RunnerConfig(epoch=3)
    assert RunnerConfig.filter_kwargs(epochs=1, bogus=2) == {"epochs": 1}
    trainer = Trainer(args=args, task="general")
    assert trainer.config.runner_config.epochs == 2 and trainer.config.optimizer.weight_decay == 0.05
    assert trainer.config.seed == 7


def test_predict_applies_the_yaml_quantization_config(tmp_path, monkeypatch):
    from mindformers_b200.modules.quantizers import QuantLinear
    from mindformers_b200.tools.register import MindFormerConfig
    from mindformers_b200.trainer.base_trainer import CausalLanguageModelingTrainer
    monkeypatch.setenv("RUN_MODE", "predict")
    cfg = MindFormerConfig({
        "run_mode": "predict", "output_dir": str(tmp_path), "save_file": str(tmp_path / "out.txt"),
        "model": {"model_config": dict(model_type="llama", num_hidden_layers=1, hidden_size=128, num_attention_heads=4,
                                       num_key_value_heads=2, intermediate_size=256, vocab_size=300,
                                       max_position_embeddings=64, params_dtype="float32")},
        "quantization_config": {"quant_method": "rtn", "weight_dtype": "int8"},
        "processor": {"tokenizer": {"type": "ByteTokenizer"}}})
    seen = {}
    import mindformers_b200.pipeline as pl
    real = pl.pipeline

    def spy(task, model, tokenizer, **kw):
        seen["model"] = model
        return real(task=task, model=model, tokenizer=tokenizer, **kw)

    monkeypatch.setattr(pl, "pipeline", spy)
    out = CausalLanguageModelingTrainer().predict(cfg, input_data=["hello"], max_new_tokens=3)
    assert out and sum(isinstance(m, QuantLinear) for m in seen["model"].modules()) == 4


def test_general_task_trainer_trains_and_scores_a_caller_supplied_network(tmp_path):
    """Any module that maps a batch to a loss: the caller's network, dataset, optimizer (or one-step wrapper) and
    metric objects go through the common loop; a missing network or dataset is an error."""
    import torch
    from mindformers_b200.core.callback import Callback
    from mindformers_b200.trainer.base_trainer import GeneralTaskTrainer

    class Classifier(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.body = torch.nn.Sequential(torch.nn.Linear(8, 16), torch.nn.Tanh(), torch.nn.Linear(16, 3))

        def forward(self, x, label=None):
            logits = self.body(x)
            if self.training:
                return torch.nn.functional.cross_entropy(logits, label)
            return logits, label

    class Accuracy:
        def clear(self):
            self.hit = self.n = 0

        def update(self, logits, label):
            self.hit += int((logits.argmax(-1) == label).sum())
            self.n += int(label.numel())

        def eval(self):
            return self.hit / max(self.n, 1)

    torch.manual_seed(0)
    w = torch.randn(8, 3)
    xs = torch.randn(256, 8)
    ys = (xs @ w).argmax(-1)
    data = [{"x": xs[i:i + 32], "label": ys[i:i + 32]} for i in range(0, 256, 32)]
    net = Classifier()
    seen = []

    class Spy(Callback):
        def on_step_end(self, ctx):
            seen.append(ctx.loss)
    trainer = GeneralTaskTrainer(model_name="common")
    metrics = {"Accuracy": Accuracy()}
    before = trainer.evaluate(network=net, dataset=data, compute_metrics=metrics)["Accuracy"]
    cfg = {"runner_config": {"epochs": 12}, "optimizer": {"type": "AdamW", "learning_rate": 0.03},
           "runner_wrapper": {"use_clip_grad": True, "max_grad_norm": 1.0}}
    from mindformers_b200.tools.register import MindFormerConfig
    ctx = trainer.train(config=MindFormerConfig(cfg), network=net, dataset=data, callbacks=[Spy()])
    assert ctx.global_step == 96 and len(seen) == 96 and seen[-1] < 0.5 * seen[0]
    after = trainer.evaluate(network=net, dataset=data, compute_metrics=metrics)["Accuracy"]
    assert after > max(before, 0.85)
    logits, _ = trainer.predict(input_data={"x": xs[:4], "label": ys[:4]}, network=net)
    assert logits.shape == (4, 3)
    # a caller-supplied optimizer, and a wrapper that does the whole step itself
    net2 = Classifier()
    opt = torch.optim.SGD(net2.parameters(), lr=0.1)
    trainer.train(network=net2, dataset=data, optimizer=opt)
    net3 = Classifier()
    opt3 = torch.optim.SGD(net3.parameters(), lr=0.1)
    calls = []

    def one_step(batch):
        opt3.zero_grad()
        loss = net3(**batch)
        loss.backward()
        opt3.step()
        calls.append(1)
        return loss
    trainer.train(network=net3, dataset=data, wrapper=one_step)
    assert len(calls) == len(data)
    with pytest.raises(NotImplementedError):
        trainer.train(dataset=data)
    with pytest.raises(NotImplementedError):
        trainer.train(network=net)
    with pytest.raises(NotImplementedError):
        trainer.evaluate(network=net, dataset=data)


def test_grouped_parameters_decay_exemptions_and_layer_wise_learning_rate():
    """Groups for group-style optimizers: 1-D parameters and biases get no weight decay; with ``layer_scale`` the learning
    rate falls by ``layer_decay`` per layer from the head down, and the replicated optimizer applies it."""
    from mindformers_b200.core.optim import ReplicatedOptimizer, build_optim
    from mindformers_b200.models import LlamaConfig, LlamaForCausalLM
    from mindformers_b200.trainer.optimizer_grouped_parameters import get_optimizer_grouped_parameters
    cfg = LlamaConfig(vocab_size=64, hidden_size=32, intermediate_size=64, num_hidden_layers=3, num_attention_heads=4,
                      num_key_value_heads=2, params_dtype="float32", compute_dtype="float32")
    torch.manual_seed(0)
    m = LlamaForCausalLM(cfg, device="cpu").model
    plain = get_optimizer_grouped_parameters(m, weight_decay=0.1)
    by_name = {g["name"]: g for g in plain}
    assert set(by_name) == {"decay", "no_decay"} and by_name["decay"]["weight_decay"] == 0.1
    assert all(p.dim() <= 1 for p in by_name["no_decay"]["params"]) and all(p.dim() > 1 for p in by_name["decay"]["params"])
    assert sum(len(g["params"]) for g in plain) == len(list(m.parameters()))
    scaled = {g["name"]: g for g in get_optimizer_grouped_parameters(m, 0.1, layer_scale=True, layer_decay=0.5)}
    assert abs(scaled["layer_0_decay"]["lr_scale"] - 0.5 ** 4) < 1e-12          # embedding
    assert abs(scaled["layer_1_decay"]["lr_scale"] - 0.5 ** 3) < 1e-12 and abs(scaled["layer_3_decay"]["lr_scale"] - 0.5) < 1e-12
    assert scaled["layer_4_decay"]["lr_scale"] == 1.0                            # output layer
    inner = build_optim({"type": "SGD", "learning_rate": 1.0, "weight_decay": 0.0, "layer_scale": True, "layer_decay": 0.5},
                        model=m)
    opt = ReplicatedOptimizer(m, inner, learning_rate=1.0, max_grad_norm=0.0)
    before = {n: p.detach().clone() for n, p in m.named_parameters()}
    for p in m.parameters():
        p.grad = torch.ones_like(p)
    opt.step()
    moved = {n: float((before[n] - p.detach()).abs().max()) for n, p in m.named_parameters()}
    assert abs(moved["embedding.word_embeddings.weight"] - 0.5 ** 4) < 1e-6
    assert abs(moved["decoder.layers.2.mlp.linear_fc2.weight"] - 0.5) < 1e-6 and abs(moved["output_layer.weight"] - 1.0) < 1e-6


def test_per_token_loss_over_micro_batches_matches_one_big_batch():
    """``calculate_per_token_loss``: micro-batches with very different numbers of target tokens; the step's gradients are
    those of (sum of token losses) / (number of target tokens of the whole step), i.e. of one big batch, and the
    denominator is taken from the batch on the device (no host read inside the step)."""
    from mindformers_b200.trainer.engine import TrainingEngine
    cfg = dict(model_type="llama", num_hidden_layers=2, hidden_size=64, num_attention_heads=4, num_key_value_heads=2,
               intermediate_size=128, vocab_size=128, rms_norm_eps=1e-5, rope_theta=10000.0, max_position_embeddings=32)
    ids = torch.randint(1, 128, (2, 33), generator=torch.Generator().manual_seed(0))
    mask = torch.ones(2, 32, dtype=torch.int32)
    mask[1, 5:] = 0                                            # the second sample has 5 target tokens, the first 32
    batch = {"input_ids": ids[:, :-1].contiguous(), "labels": ids[:, 1:].contiguous(), "loss_mask": mask}

    def run(mbs, per_token):
        torch.manual_seed(3)
        eng = TrainingEngine.from_model_config(cfg, seq_length=32, device="cpu", dtype="float32", micro_batch_size=mbs,
                                               learning_rate=1e-2, max_grad_norm=0.0, calculate_per_token_loss=per_token)
        out = eng.train_step_device(batch)
        return {n: p.detach().clone() for n, p in eng.model.named_parameters()}, float(out["loss"]), eng

    split, loss_split, eng = run(1, True)
    whole, loss_whole, _ = run(2, True)
    for n in split:
        torch.testing.assert_close(split[n], whole[n], rtol=2e-5, atol=2e-6)
    assert abs(loss_split - loss_whole) < 1e-5
    # it is NOT the mean of the per-sample means (which the default loss computes with micro batch 1)
    mean_of_means, _, _ = run(1, False)
    assert max(float((mean_of_means[n] - split[n]).abs().max()) for n in split) > 1e-5
    # the denominator stays on the device: the step never calls .item() on a tensor
    calls = []
    orig = torch.Tensor.item
    torch.Tensor.item = lambda self: (calls.append(1), orig(self))[1]
    try:
        eng.train_step_device(batch)
    finally:
        torch.Tensor.item = orig
    assert not calls


def test_only_save_strategy_writes_the_layout_and_does_not_train(tmp_path):
    from mindformers_b200.trainer import Trainer
    _fresh()
    t = Trainer(args=_cfg(tmp_path / "s", only_save_strategy=True))
    t.train()
    path = tmp_path / "s" / "strategy" / "ckpt_strategy_rank_0.json"
    info = json.load(open(path))
    assert info["tp"] == 1 and any("linear_qkv" in n for n in info["params"])
    assert not t.trainer.loss_history and not os.path.exists(tmp_path / "s" / "checkpoint")
