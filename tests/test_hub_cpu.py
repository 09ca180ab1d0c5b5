"""Dynamic modules (auto_map, REGISTER_PATH), the offline hub directory and the output mirror."""
import json
import os

import pytest
import torch

from mindformers_b200.models import AutoConfig, AutoModel
from mindformers_b200.tools.cloud_adapter import Local2ObsMonitor, mox_adapter
from mindformers_b200.tools.hub import (check_imports, get_class_from_dynamic_module, get_relative_imports,
                                        import_register_path, snapshot_download, upload_folder)
from mindformers_b200.tools.register import MindFormerModuleType, MindFormerRegister

MODEL_SRC = '''
import torch
from .configuration_toy import ToyConfig


class ToyModel(torch.nn.Module):
    config_class = ToyConfig

    def __init__(self, config, **kwargs):
        super().__init__()
        self.config = config
        self.proj = torch.nn.Linear(config.width, config.width)

    @classmethod
    def from_pretrained(cls, path, config=None, **kwargs):
        return cls(config)

    def forward(self, x):
        return self.proj(x)
'''
CONFIG_SRC = '''
class ToyConfig:
    model_type = "toy"

    def __init__(self, width=8, **kwargs):
        self.width = width

    @classmethod
    def from_dict(cls, d, **kwargs):
        return cls(**{k: v for k, v in d.items() if k == "width"})
'''


def test_auto_map_dynamic_module(tmp_path):
    (tmp_path / "modeling_toy.py").write_text(MODEL_SRC)
    (tmp_path / "configuration_toy.py").write_text(CONFIG_SRC)
    (tmp_path / "config.json").write_text(json.dumps({
        "model_type": "toy", "width": 12,
        "auto_map": {"AutoConfig": "configuration_toy.ToyConfig", "AutoModel": "modeling_toy.ToyModel"}}))
    assert get_relative_imports(str(tmp_path / "modeling_toy.py")) == ["configuration_toy"]
    cls = get_class_from_dynamic_module("modeling_toy.ToyModel", str(tmp_path))
    assert cls.__name__ == "ToyModel"
    cfg = AutoConfig.from_pretrained(str(tmp_path))
    assert type(cfg).__name__ == "ToyConfig" and cfg.width == 12
    model = AutoModel.from_pretrained(str(tmp_path))
    assert model(torch.zeros(2, 12)).shape == (2, 12)
    with pytest.raises(FileNotFoundError):
        get_class_from_dynamic_module("missing_file.Foo", str(tmp_path))
    (tmp_path / "needs_pkg.py").write_text("import surely_not_installed_pkg\n")
    with pytest.raises(ImportError):
        check_imports(str(tmp_path / "needs_pkg.py"))


def test_register_path_plugins(tmp_path, monkeypatch):
    (tmp_path / "my_plugin.py").write_text(
        "from mindformers_b200.tools.register import MindFormerRegister, MindFormerModuleType\n"
        "@MindFormerRegister.register(MindFormerModuleType.TOOLS)\n"
        "class PluggedInTool:\n    value = 41\n")
    monkeypatch.setenv("REGISTER_PATH", str(tmp_path))
    names = import_register_path()
    assert len(names) == 1
    assert MindFormerRegister.get_cls(MindFormerModuleType.TOOLS, "PluggedInTool").value == 41


def test_offline_hub_and_mirror(tmp_path, monkeypatch):
    monkeypatch.setenv("MFB200_HUB_ROOT", str(tmp_path / "hub"))
    src = tmp_path / "model"
    (src / "sub").mkdir(parents=True)
    (src / "config.json").write_text("{}")
    (src / "sub" / "w.safetensors").write_bytes(b"123")
    (src / "notes.txt").write_text("x")
    copied = upload_folder("org/toy", str(src), ignore_patterns=["*.txt"])
    assert copied == ["config.json", os.path.join("sub", "w.safetensors")]
    assert snapshot_download("org/toy") == str(tmp_path / "hub" / "org" / "toy")
    local = snapshot_download("org/toy", allow_patterns=["*.json"], local_dir=str(tmp_path / "dl"))
    assert os.listdir(local) == ["config.json"]
    with pytest.raises(FileNotFoundError):
        snapshot_download("org/absent")
    # output mirror with keep-last
    out, remote = tmp_path / "output", tmp_path / "remote"
    out.mkdir()
    (out / "a.safetensors").write_bytes(b"1")
    mon = Local2ObsMonitor(str(out), str(remote), rank_id=0, upload_frequence=2)

    class Ctx:
        cur_step_num = 2
    mon.on_step_end(Ctx())
    assert (remote / "rank_0" / "a.safetensors").exists()
    os.remove(out / "a.safetensors")
    (out / "b.safetensors").write_bytes(b"2")
    mon.on_train_end(Ctx())
    assert not (remote / "rank_0" / "a.safetensors").exists() and (remote / "rank_0" / "b.safetensors").exists()
    assert mox_adapter(str(tmp_path / "nope"), str(tmp_path / "x"), retry=1, retry_time=0) is False
