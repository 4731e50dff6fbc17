"""YAML + override loader and config validation."""
import pytest
import yaml

from areal_b200.api import cli_args as C

YAML = """
experiment_name: gsm8k-grpo
trial_name: trial0
seed: 7
cluster:
  fileroot: /tmp/areal_b200_cfgtest
  n_gpus_per_node: 8
  name_resolve: {type: memory}
gconfig:
  n_samples: 4
  max_new_tokens: 1024
rollout:
  backend: native:d4
  max_head_offpolicyness: 2
  consumer_batch_size: ${train_dataset.batch_size}
actor:
  backend: fsdp:d4
  path: /models/x
  eps_clip: 0.4
  use_decoupled_loss: true
  reward_norm: {mean_level: group, std_level: group, group_size: "${gconfig.n_samples}"}
  adv_norm: {mean_level: batch, std_level: batch}
  rejection_sampling: {metric: ratio, upper: 5.0}
  optimizer: {lr: 1.0e-5, lr_scheduler_type: constant}
  mb_spec: {max_tokens_per_mb: 10240}
ref:
  backend: ${actor.backend}
  path: ${actor.path}
train_dataset: {path: openai/gsm8k, type: rl, batch_size: 256}
saver: {freq_steps: 10}
"""


def test_load_with_overrides_and_interpolation(tmp_path):
    f = tmp_path / "c.yaml"
    f.write_text(YAML)
    cfg, path = C.load_expr_config(["--config", str(f), "actor.eps_clip=0.3", "actor.optimizer.lr=2e-6",
                                    "gconfig.n_samples=8", "+actor.c_clip=3.0", "total_train_epochs=3"], C.GRPOConfig)
    assert path == str(f)
    assert cfg.actor.eps_clip == 0.3 and cfg.actor.optimizer.lr == 2e-6 and cfg.actor.c_clip == 3.0
    assert cfg.gconfig.n_samples == 8 and cfg.actor.reward_norm.group_size == 8
    assert cfg.rollout.consumer_batch_size == 256 and cfg.ref.backend == "fsdp:d4" and cfg.ref.path == "/models/x"
    assert cfg.actor.rejection_sampling.level == "token"
    # experiment identity is propagated into sub-configs
    assert cfg.saver.experiment_name == "gsm8k-grpo" and cfg.saver.fileroot == "/tmp/areal_b200_cfgtest"
    assert cfg.actor.mb_spec.max_tokens_per_mb == 10240 and cfg.total_train_epochs == 3
    out = C.save_config(cfg, str(tmp_path / "logs"))
    assert yaml.safe_load(open(out))["actor"]["eps_clip"] == 0.3


def test_unknown_key_and_bad_values(tmp_path):
    with pytest.raises(KeyError):
        C.to_structured_cfg({"experiment_name": "a", "trial_name": "b", "actor": {"epsclip": 1}}, C.GRPOConfig)
    with pytest.raises(ValueError):
        C.NormConfig(mean_level="token")
    with pytest.raises(ValueError):
        C.PPOActorConfig(use_sapo_loss=True, use_decoupled_loss=True)
    with pytest.raises(ValueError):
        C.RejectionSamplingConfig(action="clamp", metric="kl_k1")
    with pytest.raises(ValueError):
        C.PPOActorConfig(prox_logp_method="nope")
    with pytest.raises(ValueError):
        C.AgentConfig(mode="remote")


def test_defaults_match_documented_surface():
    g = C.GenerationHyperparameters()
    assert (g.n_samples, g.max_new_tokens, g.max_tokens, g.top_p, g.temperature) == (1, 16384, 32768, 1.0, 1.0)
    a = C.PPOActorConfig()
    assert (a.ppo_n_minibatches, a.eps_clip, a.kl_ctl, a.reward_clip, a.discount, a.gae_lambda) == (4, 0.2, 0.1, 20.0, 1.0, 1.0)
    assert C.PPOCriticConfig().eps_clip == 0.5 and C.DPOEngineConfig().beta == 0.1
    assert C.MicroBatchSpec().packing_algorithm == "ffd" and C.OptimizerConfig().gradient_clipping == 1.0
    assert C.InferenceEngineConfig().max_head_offpolicyness == 0 and C.RecoverConfig().mode == "disabled"
    assert g.to_openai_args_dict()["max_completion_tokens"] == 16384 and "top_k" not in g.to_openai_args_dict()
    assert a.should_compute_prox_logp() is False
    assert C.PPOActorConfig(use_decoupled_loss=True).should_compute_prox_logp() is True
    assert C.PPOActorConfig(use_decoupled_loss=True, prox_logp_method="loglinear").should_compute_prox_logp() is False


def test_cli_reference_is_current():
    """docs/cli_reference.md is generated from the dataclasses; regenerate it when a field changes."""
    from areal_b200.tools import gen_cli_reference

    assert gen_cli_reference.main(["--check"]) == 0
