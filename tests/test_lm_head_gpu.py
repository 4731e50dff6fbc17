"""Fused LM-head logprob/entropy kernel vs log_softmax on materialised fp32 logits."""
import pytest
import torch

from areal_b200.ops import _lib
from areal_b200.ops.lm_head import lm_head_logprobs, lm_head_logprobs_ref

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("T,V,H,temp", [(1, 1000, 64, 1.0), (130, 5000, 256, 0.7), (300, 151936, 128, 1.0),
                                         (257, 4099 // 8 * 8, 512, 1.3)])
def test_lm_head_forward_backward(T, V, H, temp):
    torch.manual_seed(0)
    x = (torch.randn(T, H, device="cuda") * 0.5).bfloat16().requires_grad_()
    w = (torch.randn(V, H, device="cuda") * 0.1).bfloat16().requires_grad_()
    labels = torch.randint(0, V, (T,), device="cuda")
    logp, ent = lm_head_logprobs(x, w, labels, temp)
    assert _lib.read_status() == 0
    xr = x.detach().float().requires_grad_()
    wr = w.detach().float().requires_grad_()
    logp_r, ent_r = lm_head_logprobs_ref(xr, wr, labels, temp)
    torch.testing.assert_close(logp, logp_r, atol=2e-3, rtol=2e-3)
    torch.testing.assert_close(ent, ent_r, atol=2e-3, rtol=2e-3)
    g1 = torch.randn(T, device="cuda")
    g2 = torch.randn(T, device="cuda") * 0.1
    torch.autograd.backward([logp, ent], [g1, g2])
    torch.autograd.backward([logp_r, ent_r], [g1, g2])
    assert _lib.read_status() == 0
    def close(a, b, name):
        err = (a.float() - b).abs().max().item()
        scale = b.abs().max().item()
        assert err <= 2e-2 * scale + 1e-3, f"{name}: err {err} scale {scale}"
    close(x.grad, xr.grad, "dx")
    close(w.grad, wr.grad, "dw")


def test_fused_sampling_head_distribution_logprobs_and_greedy():
    """Gumbel-max sampling in the LM-head epilogue: the drawn tokens follow softmax(x W^T / T), the returned
    log-probability is that of the drawn token, temperature <= 0 rows take the argmax, and the device-side
    step counter gives every call fresh noise (also under CUDA-graph replay)."""
    from areal_b200.ops.lm_head import lm_head_sample, new_sampling_rng

    torch.manual_seed(0)
    H, V, B = 256, 1000, 512  # V is no multiple of the 256-column tile: the ragged edge is masked
    w = (torch.randn(V, H, device="cuda") * 0.08).bfloat16()
    x1 = torch.randn(1, H, device="cuda").bfloat16()
    x = x1.expand(B, H).contiguous()  # the same distribution in every row
    temp = torch.full((B,), 0.7, device="cuda")
    temp[:8] = 0.0  # greedy rows
    rng = new_sampling_rng(123, "cuda")
    logits = (x1.float() @ w.float().t())[0]
    ref_lp = torch.log_softmax(logits / 0.7, -1)
    counts = torch.zeros(V, device="cuda")
    draws = 0
    seen = []
    for _ in range(40):
        tok, lp = lm_head_sample(x, w, temp, rng)
        assert tok.dtype == torch.int32 and int(tok.min()) >= 0 and int(tok.max()) < V
        assert (tok[:8] == int(logits.argmax())).all()
        torch.testing.assert_close(lp[:8], torch.log_softmax(logits, -1)[tok[:8].long()], atol=2e-3, rtol=0)
        torch.testing.assert_close(lp[8:], ref_lp[tok[8:].long()], atol=2e-3, rtol=0)
        counts += torch.bincount(tok[8:].long(), minlength=V).float()
        draws += B - 8
        seen.append(tok[8:].clone())
    assert int(rng[1]) == 40
    assert not torch.equal(seen[0], seen[1]), "every call draws fresh noise"
    p = ref_lp.exp()
    # total-variation distance of the empirical distribution of ~20k draws over 1000 outcomes; the expected
    # value under exact sampling is about sum(sqrt(2 p (1-p) / (pi n))) / 2
    tv = 0.5 * (counts / draws - p).abs().sum().item()
    expect = 0.5 * torch.sqrt(2 * p * (1 - p) / (3.14159 * draws)).sum().item()
    assert tv < 1.5 * expect + 0.01, (tv, expect)
    # the head of the distribution individually: within 5 standard deviations
    top = torch.topk(p, 10).indices
    sd = torch.sqrt(p[top] * (1 - p[top]) / draws)
    assert ((counts[top] / draws - p[top]).abs() < 5 * sd + 1e-3).all()
    # rows differ inside one call (the noise depends on the row)
    assert len(torch.unique(seen[0])) > 20
    # CUDA-graph replay advances the counter on the device
    g = torch.cuda.CUDAGraph()
    s = torch.cuda.Stream()
    with torch.cuda.stream(s):
        lm_head_sample(x, w, temp, rng)
        torch.cuda.synchronize()
        with torch.cuda.graph(g, stream=s):
            tok_g, lp_g = lm_head_sample(x, w, temp, rng)
    before = int(rng[1])
    g.replay()
    a = tok_g.clone()
    g.replay()
    torch.cuda.synchronize()
    assert int(rng[1]) == before + 2 and not torch.equal(a, tok_g)
    assert _lib.read_status() == 0


def test_fused_sampling_head_at_decode_shape():
    """Qwen3-1.7B head (2048 x 151936), 300 rows (three row tiles, the last one partly filled)."""
    from areal_b200.ops.lm_head import lm_head_sample, new_sampling_rng

    torch.manual_seed(1)
    H, V, B = 2048, 151936, 300
    w = (torch.randn(V, H, device="cuda") * 0.02).bfloat16()
    x = torch.randn(B, H, device="cuda").bfloat16()
    temp = torch.ones(B, device="cuda")
    temp[::7] = 0.0
    rng = new_sampling_rng(7, "cuda")
    tok, lp = lm_head_sample(x, w, temp, rng)
    logits = x.float() @ w.float().t()
    ref = torch.log_softmax(logits, -1)
    torch.testing.assert_close(lp, ref.gather(1, tok.long()[:, None]).squeeze(1), atol=5e-3, rtol=0)
    greedy = temp <= 0
    assert torch.equal(tok[greedy].long(), logits[greedy].argmax(-1))
    # sampled rows: the drawn tokens are plausible (not stuck at the argmax, log-probabilities near the entropy)
    assert (tok[~greedy].long() != logits[~greedy].argmax(-1)).float().mean() > 0.5
    ent = -(ref.exp() * ref).sum(-1)
    assert abs(float((-lp[~greedy]).mean()) - float(ent[~greedy].mean())) < 0.5
    assert _lib.read_status() == 0
