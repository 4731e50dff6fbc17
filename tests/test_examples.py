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


def test_skypilot_task_files_parse_and_name_existing_files():
    import re

    import yaml

    files = sorted(glob.glob(os.path.join(ROOT, "examples", "skypilot", "*.sky.yaml")))
    assert len(files) == 2
    for f in files:
        task = yaml.safe_load(open(f))
        assert task["resources"]["accelerators"].startswith("B200:") and "torch.distributed.run" in task["run"]
        named = re.findall(r"(examples/[\w/.]+\.(?:py|yaml))", task["run"])
        assert len(named) == 2 and all(os.path.exists(os.path.join(ROOT, n)) for n in named), named
        # the overrides after the config path are fields of the experiment config
        overrides = [w for w in task["run"].replace("\\\n", " ").split() if "=" in w and not w.startswith("--")
                     and "$(" not in w and not w.startswith("HEAD_IP")]
        env = {k: str(v) for k, v in task.get("envs", {}).items()}
        overrides = [re.sub(r"\$(\w+)", lambda m: env.get(m.group(1), "x"), w) for w in overrides]
        cfg, _ = load_expr_config(["--config", os.path.join(ROOT, named[1])] + overrides, GRPOConfig)
        assert cfg.trial_name == "sky0"


@pytest.mark.parametrize("path", sorted(p for p in glob.glob(os.path.join(ROOT, "examples", "**", "*.yaml"), recursive=True)
                                        if not p.endswith(".sky.yaml")))
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


def _tiny_tokenizer(path):
    """A word-level tokenizer with a chat template, saved as an HF fast tokenizer (vocabulary < 1024: the tiny
    model presets). Stands in for a model directory's tokenizer, which cannot be downloaded here."""
    from tokenizers import Tokenizer, models, pre_tokenizers
    from transformers import PreTrainedTokenizerFast

    words = ["<pad>", "<eos>", "<unk>", "<|user|>", "<|assistant|>", "\\boxed{", "}", "Please", "put", "your", "final",
             "answer", "within", ".", "?", "What", "is", "plus", "minus", "times", "the", "sum", "of", "and"]
    words += [str(i) for i in range(200)]
    tok = Tokenizer(models.WordLevel({w: i for i, w in enumerate(words)}, unk_token="<unk>"))
    tok.pre_tokenizer = pre_tokenizers.WhitespaceSplit()
    fast = PreTrainedTokenizerFast(tokenizer_object=tok, pad_token="<pad>", eos_token="<eos>", unk_token="<unk>")
    fast.chat_template = ("{% for m in messages %}<|{{ m['role'] }}|> {{ m['content'] }} {% endfor %}"
                          "{% if add_generation_prompt %}<|assistant|> {% endif %}")
    fast.save_pretrained(path)
    return path


def _gsm8k_like(path, n=48):
    import json
    import random

    rnd = random.Random(0)
    os.makedirs(path, exist_ok=True)
    for split in ("train", "test"):
        with open(os.path.join(path, f"{split}.jsonl"), "w") as f:
            for _ in range(n):
                a, b = rnd.randrange(90), rnd.randrange(90)
                f.write(json.dumps({"question": f"What is {a} plus {b} ?", "answer": f"the sum #### {a + b}"}) + "\n")
    return path


def _run_example(script, yaml_name, tmp_path, extra):
    spec = importlib.util.spec_from_file_location("example_run_" + os.path.basename(script)[:-3], script)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    tok_dir = _tiny_tokenizer(str(tmp_path / "tok"))
    data_dir = _gsm8k_like(str(tmp_path / "gsm8k"))
    argv = ["--config", os.path.join(ROOT, "examples", "math", yaml_name), f"tokenizer_path={tok_dir}",
            f"train_dataset.path={data_dir}", f"cluster.fileroot={tmp_path}/exp", "trial_name=accept",
            "stats_logger.wandb.mode=disabled"] + extra
    mod.main(argv)
    return tmp_path / "exp"


def test_gsm8k_grpo_example_runs_end_to_end_on_cpu(tmp_path):
    """The GRPO example script, its CPU YAML, a local gsm8k-shaped dataset and a local tokenizer: two full
    asynchronous steps (rollout with the math reward, recompute, advantages, update, weight push), statistics
    written. Role of the reference's tests/grpo/test_grpo.py (which also asserts a reward level after real training)."""
    import json

    root = _run_example(os.path.join(ROOT, "examples", "math", "gsm8k_rl.py"), "gsm8k_grpo_cpu.yaml", tmp_path,
                        ["total_train_steps=2", "train_dataset.batch_size=4", "gconfig.max_new_tokens=8",
                         "saver.freq_epochs=null", "evaluator.freq_epochs=null"])
    logs = glob.glob(str(root / "logs" / "**" / "*.jsonl"), recursive=True)
    assert logs, "the stats logger wrote no record"
    recs = [json.loads(l) for l in open(logs[0]) if l.strip()]
    assert len(recs) >= 2 and all("step/loss" in r or any(k.endswith("actor_loss") for k in r) for r in recs)


def test_gsm8k_sft_example_runs_end_to_end_on_cpu(tmp_path):
    """The SFT example for two steps on the same local data: the loss is finite and a checkpoint appears when
    asked for (role of the reference's tests/sft/test_sft.py)."""
    script = os.path.join(ROOT, "examples", "math", "gsm8k_sft.py")
    if not os.path.exists(script):
        pytest.skip("no SFT example script")
    yamls = [y for y in ("gsm8k_sft_cpu.yaml", "gsm8k_sft.yaml") if os.path.exists(os.path.join(ROOT, "examples", "math", y))]
    if not yamls:
        pytest.skip("no SFT YAML")
    _run_example(script, yamls[0], tmp_path,
                 ["total_train_steps=2", "train_dataset.batch_size=4", "actor.model_preset=tiny-qwen2", "actor.path=",
                  "actor.init_from_scratch=true", "actor.dtype=float32", "actor.backend=fsdp:d1",
                  "valid_dataset=null", "saver.freq_epochs=null", "evaluator.freq_epochs=null"])


def test_search_agent_example_runs_end_to_end_on_cpu(tmp_path):
    """The search-agent example through the OpenAI-protocol workflow: a local QA file, a BM25 corpus, the tiny
    model (whose random text calls no tool and tags no answer, so rewards are 0) — two asynchronous steps."""
    import json

    qa_dir = tmp_path / "hotpot_qa"
    qa_dir.mkdir()
    for split in ("train", "test"):
        with open(qa_dir / f"{split}.jsonl", "w") as f:
            for i in range(16):
                f.write(json.dumps({"question": f"What is {i} plus {i} ?", "answers": [str(2 * i)]}) + "\n")
    corpus = tmp_path / "corpus.jsonl"
    corpus.write_text("\n".join(json.dumps({"id": f"d{i}", "title": f"sum {i}", "text": f"{i} plus {i} is {2 * i}"})
                                for i in range(16)))
    root = _run_example(os.path.join(ROOT, "examples", "search_agent", "search_agent_rl.py"), "gsm8k_grpo_cpu.yaml",
                        tmp_path, [f"train_dataset.path={qa_dir}", f"corpus={corpus}", "max_turns=2",
                                   "total_train_steps=2", "train_dataset.batch_size=4", "gconfig.max_new_tokens=8",
                                   "saver.freq_epochs=null", "evaluator.freq_epochs=null"])
    assert glob.glob(str(root / "logs" / "**" / "*.jsonl"), recursive=True)


def test_service_desk_example_runs_end_to_end_on_cpu(tmp_path):
    """The service-desk example through the OpenAI-protocol workflow with generated tasks and the scripted customer:
    two asynchronous steps. (The tiny model's random text calls no tool; the refusal tasks, whose reference is to
    change nothing, are the ones it can score on.)"""
    import json

    root = _run_example(os.path.join(ROOT, "examples", "service_desk", "service_desk_rl.py"), "gsm8k_grpo_cpu.yaml",
                        tmp_path, ["train_dataset.path=generate:desk:16:0", "valid_dataset=null",
                                   "total_train_steps=2", "train_dataset.batch_size=4", "gconfig.max_new_tokens=8",
                                   "saver.freq_epochs=null", "evaluator.freq_epochs=null"])
    logs = glob.glob(str(root / "logs" / "**" / "*.jsonl"), recursive=True)
    assert logs
    recs = [json.loads(l) for l in open(logs[0]) if l.strip()]
    assert len(recs) >= 2
