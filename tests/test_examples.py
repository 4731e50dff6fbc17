"""Every YAML under examples/ must load into its experiment config class, and the entry scripts
must at least import."""
import glob
import importlib.util
import os

import pytest

from areal_b200.api.cli_args import DPOConfig, GRPOConfig, RWConfig, SFTConfig, load_expr_config

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _cls(path):
    name = os.path.basename(path)
    if "sft" in name:
        return SFTConfig
    if "dpo" in name:
        return DPOConfig
    if "_rw" in name or name.startswith("rw"):
        return RWConfig
    return GRPOConfig


@pytest.mark.parametrize("path", sorted(glob.glob(os.path.join(ROOT, "examples", "**", "*.yaml"), recursive=True)))
def test_yaml_loads(path):
    cfg, _ = load_expr_config(["--config", path, "trial_name=t"], _cls(path))
    assert cfg.experiment_name and cfg.trial_name == "t"
    if hasattr(cfg, "rollout") and hasattr(cfg, "gconfig"):
        assert cfg.gconfig.n_samples >= 1


@pytest.mark.parametrize("path", sorted(glob.glob(os.path.join(ROOT, "examples", "**", "*.py"), recursive=True)))
def test_entry_script_imports(path):
    spec = importlib.util.spec_from_file_location("example_" + os.path.basename(path)[:-3], path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    assert callable(mod.main)
