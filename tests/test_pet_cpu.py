"""Parameter-efficient tuning on CPU: LoRA (zero-init equivalence, training only the adapter, merge), multi-adapter
inference, prefix tuning."""
import torch

from mindformers_b200.models import LlamaConfig, LlamaForCausalLM
from mindformers_b200.pet import (LoraConfig, LoraModel, Ptuning2Config, SLoraConfig, get_pet_model, lora_state_dict,
                                  merge_lora_weights)


def _tiny():
    cfg = LlamaConfig(vocab_size=96, hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4,
                      num_key_value_heads=2, max_position_embeddings=32, seq_length=32, params_dtype="float32",
                      compute_dtype="float32")
    torch.manual_seed(0)
    return LlamaForCausalLM(cfg, device="cpu")


def _batch():
    g = torch.Generator().manual_seed(1)
    ids = torch.randint(0, 96, (2, 17), generator=g)
    return ids[:, :-1].contiguous(), ids[:, 1:].contiguous()


def test_lora_starts_equal_trains_only_adapter_and_merges():
    base = _tiny()
    x, y = _batch()
    ref = base(x, y).item()
    model = LoraModel(LoraConfig(lora_rank=4, lora_alpha=8, target_modules=".*linear_qkv|.*linear_proj|.*linear_fc1"), base)
    assert abs(model(x, y).item() - ref) < 1e-6            # B starts at zero
    trainable = [n for n, p in model.named_parameters() if p.requires_grad]
    assert trainable and all("lora_" in n for n in trainable)
    opt = torch.optim.AdamW([p for p in model.parameters() if p.requires_grad], lr=1e-2)
    frozen_before = {n: p.clone() for n, p in model.named_parameters() if not p.requires_grad}
    for _ in range(5):
        opt.zero_grad()
        loss = model(x, y)
        loss.backward()
        opt.step()
    assert loss.item() < ref
    for n, p in model.named_parameters():
        if not p.requires_grad:
            assert torch.equal(p, frozen_before[n]), n
    tuned = model(x, y).item()
    sd = lora_state_dict(model)
    assert len(sd) == 2 * 3 * 2
    merge_lora_weights(model)
    assert abs(model(x, y).item() - tuned) < 1e-4


def test_slora_applies_adapter_per_sequence():
    base = _tiny()
    x, _ = _batch()
    net = get_pet_model(base, dict(pet_type="slora", lora_num=2, lora_rank=4, lora_alpha=8, target_modules=".*linear_proj"))
    plain = net(x).clone()
    state = {}
    for layer in net.slora.layers:
        state[f"{layer.qualified_name}.lora_a"] = torch.randn(4, layer.weight.shape[1]) * 0.1
        state[f"{layer.qualified_name}.lora_b"] = torch.randn(layer.weight.shape[0], 4) * 0.1
    net.slora.load_adapter("math", state)
    net.slora.set_adapter_ids([None, "math"], [16, 16])
    mixed = net(x)
    assert torch.allclose(mixed[:16], plain[:16], atol=1e-6)      # sequence 0: base model
    assert (mixed[16:] - plain[16:]).abs().max() > 1e-4           # sequence 1: adapter applied
    net.slora.clear()
    assert torch.allclose(net(x), plain, atol=1e-6)


def test_prefix_tuning_trains_prefix_only():
    base = _tiny()
    x, y = _batch()
    model = get_pet_model(base, Ptuning2Config(pre_seq_len=4))
    names = [n for n, p in model.named_parameters() if p.requires_grad]
    assert names and all(n.startswith("prefix_encoder") for n in names)
    opt = torch.optim.AdamW([p for p in model.parameters() if p.requires_grad], lr=5e-2)
    first = None
    for _ in range(8):
        opt.zero_grad()
        loss = model(x, y)
        first = first if first is not None else loss.item()
        loss.backward()
        opt.step()
    assert loss.item() < first


def test_slora_model_loads_adapter_table_and_routes(tmp_path):
    import json

    from safetensors.torch import save_file

    from mindformers_b200.pet.models import Ptuning2Model, SLoraModel
    from mindformers_b200.pet.pet_config import SLoraConfig as _Cfg
    torch.manual_seed(0)
    base = _tiny_model() if "_tiny_model" in globals() else None
    if base is None:
        from mindformers_b200.models import LlamaConfig, LlamaForCausalLM
        base = LlamaForCausalLM(LlamaConfig(vocab_size=64, hidden_size=32, intermediate_size=64, num_hidden_layers=2,
                                            num_attention_heads=4, num_key_value_heads=2, max_position_embeddings=32,
                                            params_dtype="float32", compute_dtype="float32")).eval()
    ids = torch.randint(0, 64, (2, 8))
    with torch.no_grad():
        plain = base(ids).clone()
    net = SLoraModel(_Cfg(lora_num=2, lora_rank=4, lora_alpha=8, target_modules=".*linear_proj"), base)
    state = {}
    for layer in net.slora.layers:
        state[f"{layer.qualified_name}.lora_a"] = torch.randn(4, layer.lora_a.shape[-1]) * 0.1
        state[f"{layer.qualified_name}.lora_b"] = torch.randn(layer.lora_b.shape[-2], 4) * 0.1
    (tmp_path / "math").mkdir()
    save_file(state, str(tmp_path / "math" / "adapter_model.safetensors"))
    (tmp_path / "lora_adapter.json").write_text(json.dumps({"math": "math"}))
    assert net.load_adapters(str(tmp_path)) == ["math"]
    with torch.no_grad():
        routed = net(ids, adapter_names=[None, "math"]).view(2, 8, -1)
        again = net(ids).view(2, 8, -1)
    plain = plain.view(2, 8, -1)
    assert torch.allclose(routed[0], plain[0], atol=1e-5) and not torch.allclose(routed[1], plain[1], atol=1e-4)
    assert torch.allclose(again, plain, atol=1e-5)                      # routing does not outlive the call
    assert issubclass(Ptuning2Model, torch.nn.Module)
