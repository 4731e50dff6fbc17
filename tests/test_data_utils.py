"""Padded/packed conversion, micro-batch splitting and padding."""
import torch

from areal_b200.api.cli_args import MicroBatchSpec
from areal_b200.utils.data import (amend_position_ids, concat_padded_tensors, pack_tensor_dict, pad_mb_list,
                                   split_padded_tensor_dict_into_mb_list, unpack_to_padded, unpad_logits)


def _batch(lens, L=None, seed=0):
    g = torch.Generator().manual_seed(seed)
    L = L or max(lens)
    B = len(lens)
    mask = torch.arange(L)[None, :] < torch.tensor(lens)[:, None]
    return dict(input_ids=torch.randint(1, 100, (B, L), generator=g) * mask, attention_mask=mask,
                loss_mask=(torch.rand(B, L, generator=g) > 0.5).int() * mask, rewards=torch.randn(B, generator=g))


def test_pack_unpack_roundtrip():
    d = _batch([3, 7, 1, 5])
    p = pack_tensor_dict(d)
    assert p["cu_seqlens"].tolist() == [0, 3, 10, 11, 16] and p["max_seqlen"] == 7
    assert p["input_ids"].shape == (16,) and p["rewards"].shape == (4,)
    assert amend_position_ids(p)["position_ids"].tolist() == [0, 1, 2, 0, 1, 2, 3, 4, 5, 6, 0, 0, 1, 2, 3, 4]
    u = unpack_to_padded(p)
    assert torch.equal(u["input_ids"], d["input_ids"]) and torch.equal(u["attention_mask"], d["attention_mask"])


def test_concat_pads_to_longest():
    a, b = _batch([2, 3]), _batch([6], seed=1)
    a["versions"] = torch.zeros(2, 3, dtype=torch.int32)
    b["versions"] = torch.ones(1, 6, dtype=torch.int32)
    c = concat_padded_tensors([a, b])
    assert c["input_ids"].shape == (3, 6) and c["rewards"].shape == (3,)
    assert c["attention_mask"][:2, 3:].sum() == 0
    assert (c["versions"][:2, 3:] == -1).all()


def test_mb_split_respects_capacity_and_restores_order():
    lens = [30, 10, 25, 5, 40, 20, 15, 35]
    d = _batch(lens)
    d["seq_id"] = torch.arange(len(lens))
    mbl = split_padded_tensor_dict_into_mb_list(d, MicroBatchSpec(max_tokens_per_mb=64))
    assert all(int(mb["cu_seqlens"][-1]) <= 64 for mb in mbl.mbs)
    assert sorted(mbl.forward_indices) == list(range(8))
    order = torch.cat([mb["seq_id"] for mb in mbl.mbs]).tolist()
    assert order == mbl.forward_indices
    assert [order[i] for i in mbl.backward_indices] == list(range(8))
    assert sum(mbl.group_lens) == 8


def test_mb_split_granularity_keeps_pairs_together():
    lens = [9, 3, 8, 2, 7, 1, 6, 4]
    d = _batch(lens)
    d["seq_id"] = torch.arange(8)
    mbl = split_padded_tensor_dict_into_mb_list(d, MicroBatchSpec(n_mbs=2, granularity=2))
    for mb in mbl.mbs:
        ids = mb["seq_id"].tolist()
        assert all(ids[i] + 1 == ids[i + 1] and ids[i] % 2 == 0 for i in range(0, len(ids), 2))


def test_pad_mb_list_alignment():
    d = _batch([100, 30, 61])
    mbl = pad_mb_list(split_padded_tensor_dict_into_mb_list(d, MicroBatchSpec(max_tokens_per_mb=128)), align_to=64)
    for mb, pad, old in zip(mbl.padded_mbs, mbl.padding_lengths, mbl.old_cu_seqlens_list):
        T = int(mb["cu_seqlens"][-1])
        assert T % 64 == 0 and T - pad == int(old[-1])
        assert mb["input_ids"].shape[0] == T
        assert unpad_logits(torch.zeros(T, 3), pad).shape[0] == int(old[-1])
