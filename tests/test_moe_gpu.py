"""MoE routing / sort / grouped-GEMM kernels against plain PyTorch fp32."""
import pytest
import torch

from areal_b200.ops import _lib, moe

pytestmark = pytest.mark.gpu


def test_route_matches_softmax_topk():
    torch.manual_seed(0)
    for T, E, k, renorm in [(37, 8, 2, True), (1000, 128, 8, True), (64, 60, 4, False)]:
        logits = torch.randn(T, E, device="cuda") * 2
        idx, w = moe.route(logits, k, renorm)
        idx_r, w_r = moe.route_ref(logits, k, renorm)
        assert torch.equal(idx.long().sort(-1).values, idx_r.long().sort(-1).values)
        assert torch.equal(idx, idx_r)  # descending score order, like topk
        torch.testing.assert_close(w, w_r, rtol=1e-5, atol=1e-6)


@pytest.mark.parametrize("T,E,k", [(5, 4, 2), (700, 8, 2), (3000, 128, 8)])
def test_sort_is_stable_and_padded(T, E, k):
    torch.manual_seed(1)
    idx = torch.stack([torch.randperm(E, device="cuda")[:k] for _ in range(T)]).int()
    if E > 2:
        idx[idx == 1] = 0  # expert 1 receives nothing (duplicates inside a row are fine for the sort)
    s = moe.sort_by_expert(idx, E)
    flat = idx.reshape(-1).long()
    counts = torch.bincount(flat, minlength=E)
    assert torch.equal(s.counts.long(), counts)
    tiles = (counts + 127) // 128
    prow0 = torch.cat([torch.zeros(1, dtype=torch.long, device="cuda"), (tiles * 128).cumsum(0)])
    assert torch.equal(s.prow0.long(), prow0)
    assert int(s.num_vm) == int(tiles.sum())
    order = torch.argsort(flat, stable=True)
    rank_in_expert = torch.empty_like(order)
    start = torch.cat([torch.zeros(1, dtype=torch.long, device="cuda"), counts.cumsum(0)])[:-1]
    rank_in_expert[order] = torch.arange(T * k, device="cuda") - start[flat[order]]
    want = prow0[flat] + rank_in_expert
    assert torch.equal(s.dest.long(), want)
    src = torch.full((s.max_rows,), -1, dtype=torch.long, device="cuda")
    src[want] = torch.arange(T * k, device="cuda")
    assert torch.equal(s.src_of.long(), src)
    te = torch.repeat_interleave(torch.arange(E, device="cuda"), tiles)
    assert torch.equal(s.tile_expert[: int(tiles.sum())].long(), te)


def _ref_fp32(x, idx, w, gate_up, down):
    T, H = x.shape
    out = torch.zeros(T, H, dtype=torch.float32, device=x.device)
    I = gate_up.shape[1] // 2
    for j in range(idx.shape[1]):
        for e in idx[:, j].unique().tolist():
            m = idx[:, j] == e
            h = x[m] @ gate_up[e].t()
            a = torch.nn.functional.silu(h[:, :I]) * h[:, I:]
            out[m] += w[m, j:j + 1] * (a @ down[e].t())
    return out


@pytest.mark.parametrize("T,E,k,H,I", [(300, 8, 2, 256, 128), (2048, 32, 4, 512, 192)])
def test_moe_experts_forward_backward(T, E, k, H, I):
    torch.manual_seed(2)
    x = torch.randn(T, H, device="cuda").bfloat16()
    gate_up = (torch.randn(E, 2 * I, H, device="cuda") * H ** -0.5).bfloat16()
    down = (torch.randn(E, H, I, device="cuda") * I ** -0.5).bfloat16()
    logits = torch.randn(T, E, device="cuda")
    logits[:, 3] = -1e9  # one expert stays empty
    idx, w = moe.route_ref(logits, k, True)
    dout = torch.randn(T, H, device="cuda").bfloat16()

    xs, ws, gs, ds = (t.clone().requires_grad_() for t in (x, w, gate_up, down))
    out = moe.moe_experts_forward(xs, idx, ws, gs, ds)
    assert _lib.read_status() == 0
    out.backward(dout)
    assert _lib.read_status() == 0

    xr, wr, gr, dr = (t.float().clone().requires_grad_() for t in (x, w, gate_up, down))
    ref = _ref_fp32(xr, idx.long(), wr, gr, dr)
    ref.backward(dout.float())

    def close(a, b, tol):
        err = (a.float() - b).abs().max().item()
        assert err <= tol * (b.abs().max().item() + 1e-6), (err, b.abs().max().item())

    close(out, ref, 2e-2)
    close(xs.grad, xr.grad, 3e-2)
    close(ws.grad, wr.grad, 3e-2)
    close(gs.grad, gr.grad, 3e-2)
    close(ds.grad, dr.grad, 3e-2)
    assert gs.grad[3].abs().max().item() == 0 and ds.grad[3].abs().max().item() == 0


def test_wgrad_accumulates_into_main_grad():
    torch.manual_seed(3)
    T, E, k, H, I = 256, 4, 2, 256, 128
    x = torch.randn(T, H, device="cuda").bfloat16().requires_grad_()
    gate_up = (torch.randn(E, 2 * I, H, device="cuda") * H ** -0.5).bfloat16().requires_grad_()
    down = (torch.randn(E, H, I, device="cuda") * I ** -0.5).bfloat16().requires_grad_()
    idx, w = moe.route_ref(torch.randn(T, E, device="cuda"), k, True)
    moe.moe_experts_forward(x, idx, w, gate_up, down).sum().backward()
    g_ref, d_ref = gate_up.grad.float().clone(), down.grad.float().clone()
    gate_up.grad = down.grad = None
    gate_up.main_grad = torch.ones(E, 2 * I, H, device="cuda")
    down.main_grad = torch.ones(E, H, I, device="cuda")
    moe.moe_experts_forward(x, idx, w, gate_up, down).sum().backward()
    assert gate_up.grad is None and down.grad is None
    torch.testing.assert_close(gate_up.main_grad - 1, g_ref, rtol=2e-2, atol=2e-2)
    torch.testing.assert_close(down.main_grad - 1, d_ref, rtol=2e-2, atol=2e-2)


def test_expert_parallel_phases_with_virtual_ranks():
    """Four virtual ep ranks on one GPU (their buffers are ordinary allocations and the phases run
    rank after rank on one stream, which stands in for the barriers): forward and backward must
    equal every rank running ALL experts on its own tokens."""
    from areal_b200.parallel.expert_parallel import EPRank

    torch.manual_seed(5)
    P, E, k, H, I = 4, 16, 2, 256, 128
    Ts = [200, 333, 64, 129]
    el = E // P
    gate_up = (torch.randn(E, 2 * I, H, device="cuda") * H ** -0.5).bfloat16()
    down = (torch.randn(E, H, I, device="cuda") * I ** -0.5).bfloat16()
    ranks = [EPRank(r, P, E, H, cap_rows=2 * sum(Ts) * k // P + 256, device=torch.device("cuda")) for r in range(P)]
    ptrs = [r.pointers() for r in ranks]
    for r in ranks:
        r.connect(ptrs)
    xs = [torch.randn(T, H, device="cuda").bfloat16() for T in Ts]
    routes = [moe.route_ref(torch.randn(T, E, device="cuda"), k, True) for T in Ts]
    douts = [torch.randn(T, H, device="cuda").bfloat16() for T in Ts]
    sorts = [moe.sort_by_expert(idx, E) for idx, _ in routes]
    counts_all = torch.stack([s.counts for s in sorts])
    plans = [r.plan(counts_all) for r in ranks]
    copy_rows = [ranks[r].dispatch(xs[r], routes[r][0].reshape(-1).contiguous(), routes[r][1].reshape(-1).contiguous(),
                                   sorts[r], plans[r]) for r in range(P)]
    saved = [ranks[r].experts_forward(plans[r], gate_up[r * el:(r + 1) * el].contiguous(),
                                      down[r * el:(r + 1) * el].contiguous()) for r in range(P)]
    outs = [ranks[r].combine(routes[r][0].reshape(-1).contiguous(), copy_rows[r], routes[r][1].reshape(-1).contiguous(),
                             Ts[r], k) for r in range(P)]
    assert _lib.read_status() == 0
    # backward
    for r in range(P):
        ranks[r].dispatch(douts[r], routes[r][0].reshape(-1).contiguous(), None, sorts[r], plans[r])
    wgrads = [ranks[r].experts_backward(saved[r], gate_up[r * el:(r + 1) * el].contiguous(),
                                        down[r * el:(r + 1) * el].contiguous()) for r in range(P)]
    dxs = [ranks[r].combine(routes[r][0].reshape(-1).contiguous(), copy_rows[r], None, Ts[r], k) for r in range(P)]
    dws = [ranks[r].pull_weight_grads(routes[r][0].reshape(-1).contiguous(), copy_rows[r]).view(Ts[r], k) for r in range(P)]
    assert _lib.read_status() == 0

    gr, dr = gate_up.float().requires_grad_(), down.float().requires_grad_()
    def close(a, b, tol=3e-2):
        err = (a.float() - b).abs().max().item()
        assert err <= tol * (b.abs().max().item() + 1e-6), (err, b.abs().max().item())
    for r in range(P):
        xr, wr = xs[r].float().requires_grad_(), routes[r][1].float().requires_grad_()
        ref = _ref_fp32(xr, routes[r][0].long(), wr, gr, dr)
        ref.backward(douts[r].float())
        close(outs[r], ref)
        close(dxs[r], xr.grad)
        close(dws[r], wr.grad)
    d_gate_up = torch.cat([g[0] for g in wgrads]).float()
    d_down = torch.cat([g[1] for g in wgrads]).float()
    close(d_gate_up, gr.grad)
    close(d_down, dr.grad)
