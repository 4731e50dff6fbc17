"""Trie packing (CPU) and tree attention on the tcgen05 kernels vs a dense ancestor-mask reference."""
import pytest
import torch

from areal_b200.ops import tree_attn as TA


def _seqs():
    p = [5, 6, 7, 8]
    return [p + [1, 2, 3], p + [1, 2, 4, 9], p + [10], p, [20, 21], [20, 22, 23]]


def test_trie_packing_shares_prefixes_and_is_depth_first():
    seqs = _seqs()
    t = TA.build_packed_tree(seqs)
    assert t.num_nodes == 4 + 3 + 2 + 1 + 1 + 3  # shared prompt, two branches sharing [1, 2], ...
    assert t.tree_cu == [0, 10, 14]
    # every sequence can be read back from its node path, positions are depths
    for s, path in zip(seqs, t.seq_nodes):
        assert [int(t.tokens[n]) for n in path] == s
        assert [int(t.position_ids[n]) for n in path] == list(range(len(s)))
    # depth-first: the interval test equals the parent-pointer walk
    m = TA.ancestor_mask(t)
    for b in range(len(t.tree_cu) - 1):
        s, e = t.tree_cu[b], t.tree_cu[b + 1]
        for i in range(s, e):
            for j in range(s, e):
                assert bool(m[i, j]) == (j <= i < s + int(t.exit[j]))
    vals = torch.arange(t.num_nodes).float()
    assert [x.tolist() for x in TA.gather_sequences(vals, t)] == [[float(n) for n in p] for p in t.seq_nodes]


def test_tree_attention_equals_per_sequence_causal_attention_cpu():
    """On the CPU path: attention over the trie gives every sequence the same outputs as ordinary
    causal attention over that sequence alone."""
    from areal_b200.ops.attention import attention_ref

    torch.manual_seed(0)
    seqs = _seqs()
    t = TA.build_packed_tree(seqs)
    H, D = 2, 16
    emb = torch.randn(30, 3, H, D)
    q, k, v = (emb[t.tokens, i] + 0.1 * t.position_ids[:, None, None] for i in range(3))
    out = TA.tree_attention(q, k, v, t)
    for s, o in zip(seqs, TA.gather_sequences(out, t)):
        ids = torch.tensor(s)
        pos = torch.arange(len(s))
        qs, ks, vs = (emb[ids, i] + 0.1 * pos[:, None, None] for i in range(3))
        torch.testing.assert_close(o, attention_ref(qs, ks, vs, [0, len(s)]), atol=1e-5, rtol=1e-5)


@pytest.mark.gpu
def test_tree_attention_kernels_forward_backward():
    torch.manual_seed(1)
    g = torch.Generator().manual_seed(3)
    prompt_a = torch.randint(0, 1000, (300,), generator=g).tolist()
    prompt_b = torch.randint(0, 1000, (70,), generator=g).tolist()
    seqs = [prompt_a + torch.randint(0, 1000, (int(n),), generator=g).tolist() for n in (200, 37, 450, 129)]
    seqs += [prompt_b + torch.randint(0, 1000, (int(n),), generator=g).tolist() for n in (64, 1)]
    seqs.append(seqs[0][:420] + [7, 7, 7])  # a deeper branch point
    t = TA.build_packed_tree(seqs)
    N, Hq, Hkv, D = t.num_nodes, 4, 2, 128
    q = torch.randn(N, Hq, D, device="cuda").bfloat16().requires_grad_()
    k = torch.randn(N, Hkv, D, device="cuda").bfloat16().requires_grad_()
    v = torch.randn(N, Hkv, D, device="cuda").bfloat16().requires_grad_()
    do = torch.randn(N, Hq, D, device="cuda").bfloat16()
    out = TA.tree_attention(q, k, v, t)
    out.backward(do)
    from areal_b200.ops import _lib

    assert _lib.read_status() == 0
    qr, kr, vr = (x.detach().float().requires_grad_() for x in (q, k, v))
    ref = TA.tree_attention_ref(qr, kr, vr, t)
    ref.backward(do.float())
    torch.testing.assert_close(out.float(), ref, atol=3e-2, rtol=3e-2)
    for a, b in ((q.grad, qr.grad), (k.grad, kr.grad), (v.grad, vr.grad)):
        err = (a.float() - b).abs().max().item()
        assert err <= 3e-2 * b.abs().max().item() + 2e-2, err
