"""Tensor parallelism (sequence-parallel activations, vocab-parallel head), Ulysses sequence
parallelism and their combinations with data parallelism: one optimizer step on gloo ranks
must reproduce the single-process loss, gradient norm and every gradient."""
import os
import subprocess
import sys

import pytest

from tests.conftest import free_port

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
WORKER = os.path.join(ROOT, "tests", "torchrun", "run_model_parallel.py")


def _ref(tmp_path, critic=False, n_mbs=1, preset="tiny-qwen2", images=False, extra=()):
    f = str(tmp_path / ("ref_c.pt" if critic else "ref.pt"))
    cmd = [sys.executable, WORKER, "--ref", "--n-mbs", str(n_mbs), "--preset", preset, f] + (["--critic"] if critic else [])
    cmd += (["--images"] if images else []) + list(extra)
    env = {k: v for k, v in os.environ.items() if k not in ("RANK", "WORLD_SIZE", "LOCAL_RANK")}
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    return f


def _run(n, port, args, ref):
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}",
           "--master-addr", "127.0.0.1", "--master-port", str(free_port()), WORKER] + args + [ref]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0 and "OK" in r.stdout, r.stdout[-2000:] + r.stderr[-3000:]


@pytest.mark.parametrize("n,args", [(2, ["--tp", "2"]), (2, ["--sp", "2"]), (4, ["--tp", "2", "--sp", "2"]),
                                    (4, ["--tp", "2"])])
def test_lm_step_matches_single_process(tmp_path, n, args):
    _run(n, 29640 + n + len(args), args, _ref(tmp_path))


def test_zigzag_context_parallel_matches_single_process(tmp_path):
    """cp 2 with zig-zag chunks and gathered K/V (sequences padded to 2 * cp * 128 tokens inside)."""
    _run(2, 29655, ["--sp", "2", "--zigzag"], _ref(tmp_path))


def test_critic_step_matches_single_process(tmp_path):
    _run(2, 29651, ["--tp", "2", "--critic"], _ref(tmp_path, critic=True))


@pytest.mark.parametrize("n,args", [(2, ["--pp", "2"]), (4, ["--pp", "2", "--tp", "2"])])
def test_pipeline_step_matches_single_process(tmp_path, n, args):
    """Two micro-batches through a two-stage pipeline (alone and with tensor parallelism inside
    each stage)."""
    _run(n, 29660 + n, args + ["--n-mbs", "2"], _ref(tmp_path, n_mbs=2))


@pytest.mark.parametrize("n,ep", [(2, 2), (4, 2)])
def test_expert_parallel_step_matches_single_process(tmp_path, n, ep):
    """MoE model with the experts split over the ep group (tokens gathered / partial outputs summed
    on gloo; expert weights in their own flat buffer, clipped by the joint gradient norm)."""
    _run(n, 29670 + n, ["--ep", str(ep), "--preset", "tiny-qwen3-moe"], _ref(tmp_path, preset="tiny-qwen3-moe"))


@pytest.mark.parametrize("n,args", [(2, ["--tp", "2", "--ep", "2"]), (4, ["--tp", "2", "--ep", "2"]),
                                    (4, ["--tp", "2", "--ep", "4"]), (4, ["--tp", "2", "--pp", "2", "--ep", "2", "--n-mbs", "2"]),
                                    (4, ["--pp", "2", "--ep", "2", "--n-mbs", "2"]),
                                    (2, ["--tp", "2", "--etp", "2"]), (4, ["--tp", "2", "--ep", "2", "--etp", "2"]),
                                    (4, ["--tp", "2", "--etp", "2"])])
def test_hybrid_tensor_and_expert_parallel_step_matches_single_process(tmp_path, n, args):
    """Attention tensor-parallel, experts spread over the same ranks (the ``(attn:..t2|ffn:..e2)`` layout): the
    token slices that sequence-parallel activations leave on the tensor-parallel ranks are exchanged for experts;
    expert-parallel groups may also span several tensor-parallel groups, and pipeline stages (whose experts all
    count in the clipping norm). ``--etp``: expert tensor parallelism, the ranks of a group hold slices of the same
    experts, pool their tokens and sum their partial outputs."""
    n_mbs = 2 if "--n-mbs" in args else 1
    _run(n, 29742 + n + 3 * len(args), args + ["--preset", "tiny-qwen3-moe"],
         _ref(tmp_path, preset="tiny-qwen3-moe", n_mbs=n_mbs))


@pytest.mark.parametrize("n,pp,ep,tp,etp,preset", [(2, 1, 2, 2, 1, "tiny-qwen3-moe"), (4, 2, 2, 2, 1, "tiny-qwen3-moe"),
                                                   (4, 1, 4, 2, 1, "tiny-qwen3-moe"), (2, 1, 1, 2, 2, "tiny-qwen3-moe"),
                                                   (4, 1, 2, 2, 2, "tiny-qwen3-moe"),
                                                   # latent attention split by head, a replicated shared expert
                                                   (2, 1, 2, 2, 1, "tiny-deepseek-v3"), (4, 2, 2, 2, 1, "tiny-deepseek-v3")])
def test_checkpoint_under_the_hybrid_layout(tmp_path, n, pp, ep, tp, etp, preset):
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}", "--master-addr",
           "127.0.0.1", "--master-port", str(free_port()),
           os.path.join(ROOT, "tests", "torchrun", "run_vl_tp_hf.py"),
           preset, str(pp), str(tmp_path / "ckpt"), str(ep), str(tp), str(etp)]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0 and "OK" in r.stdout, r.stdout[-2000:] + r.stderr[-3000:]


@pytest.mark.parametrize("n,args", [(2, ["--pp", "2"]), (4, ["--pp", "2"]), (2, ["--tp", "2"]),
                                    (4, ["--tp", "2", "--pp", "2"]), (4, ["--tp", "2"])])
def test_lora_step_under_model_parallelism_matches_single_process(tmp_path, n, args):
    """Adapters on every dense projection, base frozen: the adapter gradients (both factors; B is given non-zero
    values that depend only on the parameter's global name), the loss and the clipping norm over all stages. Under
    tensor parallelism the adapter of a column-parallel projection gathers the token slices and keeps B by rows, that
    of a row-parallel projection keeps A by columns and sums / scatters the rank-sized partial products."""
    _run(n, 0, args + ["--lora", "--n-mbs", "2", "--preset", "tiny-qwen2-4l"],
         _ref(tmp_path, preset="tiny-qwen2-4l", n_mbs=2, extra=["--lora"]))


def test_mixture_layers_under_tensor_parallelism_need_expert_parallelism():
    from areal_b200.models.config import PRESETS
    from areal_b200.models.qwen import build_model
    from areal_b200.parallel.context import ParallelContext

    with pytest.raises(NotImplementedError, match="e = t"):
        build_model(PRESETS["tiny-qwen3-moe"], seed=None, pctx=ParallelContext(tp_size=2, tp_rank=0))


@pytest.mark.parametrize("n,preset,extra", [(2, "tiny-qwen2_5-vl", []), (2, "tiny-qwen3-vl", ["--shard-vision"]),
                                            (4, "tiny-qwen3-vl", ["--n-mbs", "2"]),
                                            (2, "tiny-qwen2_5-vl", ["--shard-vision", "--one-image"])])
def test_vision_language_step_under_ulysses(tmp_path, n, preset, extra):
    """Image prompts under Ulysses sequence parallelism (image features and the per-token rotary table built for
    the whole micro-batch, the decoder on this rank's rows; optionally the tower's images divided over the ranks):
    same loss and gradients, vision tower included, as one process."""
    n_mbs = 2 if "--n-mbs" in extra else 1
    _run(n, 29680 + n + len(extra), ["--sp", "2", "--preset", preset, "--images"] + extra,
         _ref(tmp_path, preset=preset, images=True, n_mbs=n_mbs,
              extra=["--one-image"] if "--one-image" in extra else []))


@pytest.mark.parametrize("n,preset,par", [(2, "tiny-qwen2_5-vl", ["--tp", "2"]),
                                          (4, "tiny-qwen3-vl", ["--tp", "2", "--sp", "2", "--shard-vision"])])
def test_vision_language_step_under_tensor_parallelism(tmp_path, n, preset, par):
    """Image prompts with a tensor-parallel decoder (vocab-parallel embedding, token-sharded activations: the
    image rows of this rank's tokens get their features; the tower is replicated and its gradients are summed
    over the group), alone and combined with Ulysses."""
    _run(n, 29690 + n, par + ["--preset", preset, "--images"], _ref(tmp_path, preset=preset, images=True))


@pytest.mark.parametrize("n,args", [(2, ["--ep", "2"]), (2, ["--sp", "2"]), (2, ["--pp", "2", "--n-mbs", "2"]),
                                    (2, ["--tp", "2", "--ep", "2"]), (2, ["--tp", "2", "--etp", "2"]),
                                    (4, ["--tp", "2", "--ep", "2", "--pp", "2", "--n-mbs", "2"])])
def test_latent_attention_family_step_matches_single_process(tmp_path, n, args):
    """DeepSeek-V3 architecture (latent attention, grouped sigmoid routing, ungated shared expert, dense first
    layer) under expert, Ulysses, pipeline and tensor parallelism (bottlenecks replicated, heads split, the shared
    rotary key gathered; experts over the tensor-parallel ranks)."""
    _run(n, 0, args + ["--preset", "tiny-deepseek-v3"], _ref(tmp_path, preset="tiny-deepseek-v3", n_mbs=2))


def test_lightning_attention_refuses_tensor_parallelism():
    import torch

    from areal_b200.models.config import PRESETS
    from areal_b200.models.qwen import build_model
    from areal_b200.parallel.context import ParallelContext

    with pytest.raises(NotImplementedError, match="tensor parallelism"):
        build_model(PRESETS["tiny-bailing-hybrid"], dtype=torch.float32, seed=None,
                    pctx=ParallelContext(tp_size=2, tp_rank=0, ep_size=2))


@pytest.mark.parametrize("n,pp,preset,ep", [(2, 1, "tiny-qwen3-vl", 1), (4, 2, "tiny-qwen3-vl", 1),
                                            (2, 2, "tiny-qwen2", 1), (2, 1, "tiny-qwen3-moe", 2),
                                            (2, 2, "tiny-deepseek-v3", 1), (2, 1, "tiny-deepseek-v3", 2),
                                            (2, 2, "tiny-bailing-hybrid", 1), (2, 1, "tiny-bailing-hybrid", 2)])
def test_checkpoint_under_tensor_pipeline_and_expert_parallelism(tmp_path, n, pp, preset, ep):
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}", "--master-addr",
           "127.0.0.1", "--master-port", str(free_port()), os.path.join(ROOT, "tests", "torchrun", "run_vl_tp_hf.py"),
           preset, str(pp), str(tmp_path / "ckpt"), str(ep)]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0 and "OK" in r.stdout, r.stdout[-2000:] + r.stderr[-3000:]


@pytest.mark.parametrize("n,preset,par", [(2, "tiny-qwen3-vl", ["--pp", "2"]), (4, "tiny-qwen2_5-vl", ["--pp", "2", "--tp", "2"])])
def test_vision_language_step_under_pipeline_parallelism(tmp_path, n, preset, par):
    """The tower and the deep-stack adds live on the first stage; later stages rebuild only the rotary table."""
    _run(n, 29705 + n, par + ["--preset", preset, "--images", "--n-mbs", "2"],
         _ref(tmp_path, preset=preset, images=True, n_mbs=2))
