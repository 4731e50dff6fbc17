"""Checked mode: host-side validation of data-dependent kernel indices and operand layouts."""
import pytest
import torch

from areal_b200.ops import _lib


def test_check_index_ranges():
    t = torch.tensor([0, 3, 7])
    _lib.check_index("site", t, 8)
    with pytest.raises(_lib.KernelArgumentError, match=r"site: index range \[0, 7\] outside \[0, 7\)"):
        _lib.check_index("site", t, 7)
    with pytest.raises(_lib.KernelArgumentError):
        _lib.check_index("site", torch.tensor([-1, 2]), 8)
    _lib.check_index("site", torch.tensor([-1, 2]), 8, allow_negative=True)      # the kernel skips negatives
    _lib.check_index("site", torch.tensor([9, 2]), 8, where=torch.tensor([False, True]))
    _lib.check_index("site", torch.empty(0, dtype=torch.long), 1)
    _lib.check_index("site", None, 1)


def test_check_operand_layout():
    x = torch.zeros(4, 8, dtype=torch.bfloat16)
    _lib.check_operand("x", x, torch.bfloat16, (4, None))
    with pytest.raises(_lib.KernelArgumentError, match="dtype"):
        _lib.check_operand("x", x, torch.float32)
    with pytest.raises(_lib.KernelArgumentError, match="shape"):
        _lib.check_operand("x", x, None, (4, 9))
    with pytest.raises(_lib.KernelArgumentError, match="contiguous"):
        _lib.check_operand("x", x.t())
    with pytest.raises(_lib.KernelArgumentError, match="aligned"):
        _lib.check_operand("x", x.view(-1)[1:], align=16)


def test_checked_is_off_by_default(monkeypatch):
    monkeypatch.delenv("AREAL_B200_CHECKED", raising=False)
    assert not _lib.checked()
    monkeypatch.setenv("AREAL_B200_CHECKED", "1")
    assert _lib.checked()


@pytest.mark.gpu
def test_wrappers_reject_bad_indices_before_launch(monkeypatch):
    """Every rejected call raises on the host: no kernel is launched with the bad argument."""
    from areal_b200.ops import fused, moe, rollout_ops

    monkeypatch.setenv("AREAL_B200_CHECKED", "1")
    dev = "cuda"
    Hq, Hkv, D, T = 4, 2, 128, 16
    qkv = torch.randn(T, (Hq + 2 * Hkv) * D, device=dev, dtype=torch.bfloat16)
    cos, sin = fused.rope_tables(32, D, 1e4, dev)
    pos = torch.arange(T, device=dev, dtype=torch.int32)
    before = _lib.checks_run()
    q, k, v = fused.qknorm_rope(qkv, None, None, cos, sin, pos, Hq, Hkv, D)
    assert _lib.checks_run() > before
    ref = fused.qknorm_rope_ref(qkv, None, None, cos, sin, pos, Hq, Hkv, D, 1e-6)
    assert torch.allclose(q.float(), ref[0].float(), atol=2e-2)
    with pytest.raises(_lib.KernelArgumentError, match="pos"):
        fused.qknorm_rope(qkv, None, None, cos, sin, pos + 20, Hq, Hkv, D)      # reaches past the 32-row table

    nb, bs, B = 8, 16, 2
    kc = torch.randn(nb, Hkv, bs, D, device=dev, dtype=torch.bfloat16)
    vc = torch.randn_like(kc)
    qd = torch.randn(B, Hq, D, device=dev, dtype=torch.bfloat16)
    bt = torch.tensor([[0, 1, 99, 99], [2, 3, 4, 99]], device=dev, dtype=torch.int32)   # 99: unused entries
    lens = torch.tensor([20, 40], device=dev, dtype=torch.int32)
    out = rollout_ops.paged_decode(qd, kc, vc, bt, lens)
    assert torch.allclose(out.float(), rollout_ops.paged_decode_ref(qd, kc, vc, bt, lens).float(), atol=3e-2)
    with pytest.raises(_lib.KernelArgumentError, match="block_table"):
        rollout_ops.paged_decode(qd, kc, vc, bt, torch.tensor([20, 50], device=dev, dtype=torch.int32))
    with pytest.raises(_lib.KernelArgumentError, match="seq_lens"):
        rollout_ops.paged_decode(qd, kc, vc, bt, torch.tensor([20, 65], device=dev, dtype=torch.int32))
    slots = torch.tensor([0, 5, -1, nb * bs], device=dev)
    with pytest.raises(_lib.KernelArgumentError, match="slot_mapping"):
        rollout_ops.kv_cache_write(kc[0, :, :4].transpose(0, 1).contiguous(), vc[0, :, :4].transpose(0, 1).contiguous(),
                                   slots, kc, vc)
    idx = torch.tensor([[0, 3], [2, 4]], device=dev, dtype=torch.int32)
    with pytest.raises(_lib.KernelArgumentError, match="expert_ids"):
        moe.sort_by_expert(idx, 4)
    assert int(moe.sort_by_expert(idx, 5).counts.sum()) == 4
    assert _lib.read_status() == 0
