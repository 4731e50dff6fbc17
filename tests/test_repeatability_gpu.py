"""Race and overrun detectors that need no tool: every kernel run twice on the same inputs must give the
same bits (an inter-CTA race or an uninitialised read shows up as a difference), and outputs placed between
guard rows of a known pattern must leave the guards untouched (an out-of-bounds store shows up as a damaged
guard). Shapes are ragged on purpose: the last tile of every dimension is partly filled."""
import pytest
import torch

from areal_b200.ops import _lib
from areal_b200.ops.attention import VarlenMeta, varlen_attention
from areal_b200.ops.gemm import gemm
from areal_b200.ops.lm_head import lm_head_logprobs

pytestmark = pytest.mark.gpu

CANARY = 12345.0


def _guarded(rows, cols, dtype, guard=8):
    buf = torch.full((rows + 2 * guard, cols), CANARY, dtype=dtype, device="cuda")
    return buf, buf[guard:guard + rows]


def _guards_intact(buf, rows, guard=8):
    return bool((buf[:guard] == CANARY).all() and (buf[guard + rows:] == CANARY).all())


@pytest.mark.parametrize("M,N,K", [(130, 264, 200), (1000, 520, 1032), (257, 136, 72)])
def test_gemm_is_repeatable_and_stays_inside_its_output(M, N, K):
    torch.manual_seed(0)
    a = torch.randn(M, K, device="cuda").bfloat16()
    b = torch.randn(N, K, device="cuda").bfloat16()
    buf1, out1 = _guarded(M, N, torch.bfloat16)
    buf2, out2 = _guarded(M, N, torch.bfloat16)
    gemm(a, b, out=out1)
    gemm(a, b, out=out2)
    torch.cuda.synchronize()
    assert torch.equal(out1, out2)
    assert _guards_intact(buf1, M) and _guards_intact(buf2, M)
    torch.testing.assert_close(out1.float(), a.float() @ b.float().t(), atol=0.5, rtol=2e-2)
    # fp32 accumulation target (the weight-gradient path)
    bufg, g = _guarded(N, K, torch.float32)
    g.zero_()
    dy = torch.randn(M, N, device="cuda").bfloat16()
    gemm(dy, a, a_mn=True, b_mn=True, out=g, accumulate=True)
    first = g.clone()
    g.zero_()
    gemm(dy, a, a_mn=True, b_mn=True, out=g, accumulate=True)
    assert torch.equal(first, g) and _guards_intact(bufg, N)


def test_attention_forward_and_dk_dv_are_repeatable_dq_under_deterministic_mode():
    from areal_b200.utils.determinism import set_deterministic_algorithms

    torch.manual_seed(1)
    lens = [257, 130, 700, 64, 1]
    cu = [0]
    for L in lens:
        cu.append(cu[-1] + L)
    T, Hq, Hkv, D = cu[-1], 4, 2, 128
    meta = VarlenMeta(cu, torch.device("cuda"))
    q = torch.randn(T, Hq, D, device="cuda").bfloat16()
    k = torch.randn(T, Hkv, D, device="cuda").bfloat16()
    v = torch.randn(T, Hkv, D, device="cuda").bfloat16()
    do = torch.randn(T, Hq, D, device="cuda").bfloat16()

    def run():
        qq, kk, vv = (t.clone().requires_grad_() for t in (q, k, v))
        o = varlen_attention(qq, kk, vv, meta)
        o.backward(do)
        return o.detach(), qq.grad, kk.grad, vv.grad

    o1, dq1, dk1, dv1 = run()
    o2, dq2, dk2, dv2 = run()
    assert torch.equal(o1, o2) and torch.equal(dk1, dk2) and torch.equal(dv1, dv2)
    torch.testing.assert_close(dq1.float(), dq2.float(), atol=2e-2, rtol=2e-2)  # fp32 atomics: order may differ
    set_deterministic_algorithms(True)
    try:
        _, dq3, dk3, dv3 = run()
        _, dq4, dk4, dv4 = run()
        assert torch.equal(dq3, dq4) and torch.equal(dk3, dk4) and torch.equal(dv3, dv4)
        torch.testing.assert_close(dq3.float(), dq1.float(), atol=3e-2, rtol=3e-2)
        torch.testing.assert_close(dk3.float(), dk1.float(), atol=3e-2, rtol=3e-2)
    finally:
        set_deterministic_algorithms(False)
    assert _lib.read_status() == 0


def test_lm_head_statistics_are_repeatable():
    torch.manual_seed(2)
    T, V, H = 333, 5003 // 8 * 8, 256
    x = (torch.randn(T, H, device="cuda") * 0.5).bfloat16()
    w = (torch.randn(V, H, device="cuda") * 0.1).bfloat16()
    labels = torch.randint(0, V, (T,), device="cuda")
    a = lm_head_logprobs(x, w, labels, 1.0)
    b = lm_head_logprobs(x, w, labels, 1.0)
    assert torch.equal(a[0], b[0]) and torch.equal(a[1], b[1])


def test_moe_dispatch_and_grouped_gemm_are_repeatable():
    from areal_b200.ops import moe as moe_ops

    torch.manual_seed(3)
    T, H, E, I, k = 517, 256, 8, 128, 2
    x = torch.randn(T, H, device="cuda").bfloat16()
    gate_up = (torch.randn(E, 2 * I, H, device="cuda") * 0.05).bfloat16()
    down = (torch.randn(E, H, I, device="cuda") * 0.05).bfloat16()
    logits = torch.randn(T, E, device="cuda")
    ids, wts = moe_ops.route(logits, k, True)
    y1 = moe_ops.moe_experts_forward(x, ids, wts, gate_up, down)
    y2 = moe_ops.moe_experts_forward(x, ids, wts, gate_up, down)
    assert torch.equal(y1, y2)
    ref = moe_ops.moe_experts_ref(x, ids, wts, gate_up, down)
    torch.testing.assert_close(y1.float(), ref.float(), atol=3e-2, rtol=3e-2)
    assert _lib.read_status() == 0
