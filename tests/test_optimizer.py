"""Sharded optimizer rules (AdamW fp32, AdamW with bf16 state + Kahan compensation, SGD) against
torch.optim on the same gradients; the CUDA kernels against the same oracle."""
import pytest
import torch

from areal_b200.api.cli_args import OptimizerConfig
from areal_b200.engine.flat_params import FlatParams, ShardedAdamW


class _Toy(torch.nn.Module):
    def __init__(self, dtype, device):
        super().__init__()
        g = torch.Generator().manual_seed(0)
        self.a = torch.nn.Parameter(torch.randn(37, 24, generator=g).to(dtype).to(device))
        self.b = torch.nn.Parameter(torch.randn(131, generator=g).to(dtype).to(device))


def _run(kind, device, dtype, steps=20, lr=1e-2, wd=0.1, clip=0.0):
    m = _Toy(dtype, device)
    ref = [p.detach().float().cpu().clone().requires_grad_(True) for p in (m.a, m.b)]
    cfg = OptimizerConfig(type=kind, lr=lr, weight_decay=wd, warmup_steps_proportion=0.0, gradient_clipping=clip)
    flat = FlatParams(m, "local")
    opt = ShardedAdamW(flat, cfg, total_steps=steps)
    if kind == "sgd":
        topt = torch.optim.SGD(ref, lr=lr, weight_decay=wd)
    else:
        topt = torch.optim.AdamW(ref, lr=lr, weight_decay=wd, betas=(cfg.beta1, cfg.beta2), eps=cfg.eps)
    g = torch.Generator().manual_seed(1)
    for _ in range(steps):
        grads = [torch.randn(p.shape, generator=g) * 0.1 for p in ref]
        for p, r, gr in zip((m.a, m.b), ref, grads):
            p.main_grad.copy_(gr.to(device))
            r.grad = gr.clone()
        if clip > 0:
            torch.nn.utils.clip_grad_norm_(ref, clip)
        st = opt.step()
        topt.step()
        assert st["update_successful"] == 1.0
    return [p.detach().float().cpu() for p in (m.a, m.b)], [r.detach() for r in ref], opt


@pytest.mark.parametrize("kind", ["adam", "sgd"])
def test_fp32_rules_match_torch(kind):
    got, want, _ = _run(kind, "cpu", torch.float32, clip=0.5)
    for a, b in zip(got, want):
        assert torch.allclose(a, b, atol=2e-5, rtol=1e-4)


def test_bf16_state_adamw_tracks_fp32():
    got, want, opt = _run("adam_bf16", "cpu", torch.bfloat16, steps=40)
    assert opt.master.dtype == opt.exp_avg.dtype == opt.exp_avg_sq.dtype == torch.bfloat16
    for a, b in zip(got, want):
        assert (a - b).abs().max() < 0.03


def test_kahan_compensation_keeps_small_updates():
    """Updates far below one bf16 ulp of the weight vanish without compensation and accumulate with it."""
    m = _Toy(torch.bfloat16, "cpu")
    with torch.no_grad():
        m.a.fill_(1.0)
        m.b.fill_(1.0)
    flat = FlatParams(m, "local")
    opt = ShardedAdamW(flat, OptimizerConfig(type="adam_bf16", lr=1e-4, weight_decay=0.0, warmup_steps_proportion=0.0,
                                             gradient_clipping=0.0), total_steps=100)
    for _ in range(100):
        m.a.main_grad.fill_(1.0)
        m.b.main_grad.fill_(1.0)
        opt.step()
    # 100 steps of -1e-4 each (|g|/sqrt(g²) = 1): 1 - 0.01; one bf16 ulp at 1.0 is 0.0078
    assert abs(float(m.b.detach()[0]) + float(opt.master[flat.entries[1][2]]) - 0.99) < 2e-3
    assert float(m.b.detach()[0]) < 1.0


@pytest.mark.gpu
@pytest.mark.parametrize("kind", ["adam", "adam_bf16", "sgd"])
def test_cuda_kernels_match_torch(kind):
    got, want, _ = _run(kind, "cuda", torch.bfloat16, steps=30, clip=0.5)
    for a, b in zip(got, want):
        # weights are published in bf16: one ulp of the largest weights (~4) is 0.03
        assert (a - b).abs().max() < (0.05 if kind == "adam_bf16" else 0.02)


@pytest.mark.gpu
def test_host_resident_state_streams_to_the_same_result():
    """Master weights and moments in pinned host memory, streamed through the GPU in chunks
    (several chunks, staging slots reused): bitwise the same weights as device-resident state."""
    def run(host):
        m = _Toy(torch.bfloat16, "cuda")
        big = torch.nn.Parameter(torch.randn(70001, generator=torch.Generator().manual_seed(3)).to(torch.bfloat16).cuda())
        m.big = big
        cfg = OptimizerConfig(type="adam", lr=1e-2, weight_decay=0.1, warmup_steps_proportion=0.0, gradient_clipping=0.5)
        flat = FlatParams(m, "local")
        opt = ShardedAdamW(flat, cfg, total_steps=5, host_state=host, prefetch=1, chunk_numel=8192)
        g = torch.Generator().manual_seed(1)
        for _ in range(5):
            flat.main_grad.copy_((torch.randn(flat.numel, generator=g) * 0.1).cuda())
            assert opt.step()["update_successful"] == 1.0
        return flat.flat.clone(), opt

    w_dev, _ = run(False)
    w_host, opt = run(True)
    assert opt.host_state and opt.master.is_pinned() and not opt.master.is_cuda
    assert torch.equal(w_dev, w_host)
