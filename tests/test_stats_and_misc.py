"""Stats tracker, frequency control, name resolve, seeding."""
import time

import pytest
import torch

from areal_b200.api.cli_args import NameResolveConfig
from areal_b200.utils import name_resolve, seeding, stats_tracker
from areal_b200.utils.stats_tracker import DistributedStatsTracker, ReduceType
from areal_b200.utils.timeutil import EpochStepTimeFreqCtl, FrequencyControl


def test_tracker_masked_stats_and_scopes():
    t = DistributedStatsTracker()
    mask = torch.tensor([[True, False], [True, True]])
    with t.scope("actor"):
        t.denominator(n_tokens=mask)
        t.stat(loss=torch.tensor([[1.0, 100.0], [2.0, 6.0]]), denominator="n_tokens")
        t.stat(kl=torch.tensor([[1.0, 100.0], [3.0, 5.0]]), denominator="n_tokens", reduce_type=ReduceType.SUM)
        t.scalar(lr=0.5)
        t.scalar(lr=1.5)
    out = t.export()
    assert out["actor/loss/avg"] == pytest.approx(3.0) and out["actor/loss/min"] == 1.0 and out["actor/loss/max"] == 6.0
    assert out["actor/n_tokens"] == 3.0 and out["actor/kl"] == 9.0
    assert out["actor/lr"] == 1.0 and out["actor/lr__count"] == 2.0
    assert t.export() == {}
    with pytest.raises(ValueError):
        t.stat(x=torch.ones(2), denominator="missing")
    with pytest.raises(ValueError):
        t.denominator(bad=torch.ones(2))


def test_tracker_accumulates_over_microbatches_and_merges_workers():
    t = DistributedStatsTracker()
    for vals, m in (([1.0, 3.0], [True, True]), ([10.0], [True])):
        t.denominator(n=torch.tensor(m))
        t.stat(v=torch.tensor(vals), denominator="n")
    out = t.export()
    assert out["v/avg"] == pytest.approx(14 / 3) and out["n"] == 3
    merged = stats_tracker.merge_scalar_stats([{"r": 1.0, "r__count": 1.0}, {"r": 4.0, "r__count": 3.0}])
    assert merged["r"] == pytest.approx(3.25) and merged["r__count"] == 4.0


def test_frequency_controls():
    f = FrequencyControl(frequency_steps=3)
    assert [f.check() for _ in range(7)] == [False, False, True, False, False, True, False]
    c = EpochStepTimeFreqCtl(freq_epoch=None, freq_step=2, freq_sec=None)
    assert [c.check(0, 1) for _ in range(4)] == [False, True, False, True]
    e = EpochStepTimeFreqCtl(freq_epoch=1, freq_step=None, freq_sec=None)
    assert [e.check(int(i == 2), 1) for i in range(4)] == [False, False, True, False]
    s = EpochStepTimeFreqCtl(None, None, 0.05)
    assert s.check(0, 1) is False
    time.sleep(0.07)
    assert s.check(0, 1) is True
    st = c.state_dict()
    c2 = EpochStepTimeFreqCtl(None, 2, None)
    c2.load_state_dict(st)
    assert c2.check(0, 1) == c.check(0, 1)


@pytest.mark.parametrize("kind", ["memory", "nfs"])
def test_name_resolve(kind, tmp_path):
    repo = name_resolve.make_repository(NameResolveConfig(type=kind, nfs_record_root=str(tmp_path)))
    repo.add("exp/t/gen_servers/0", "10.0.0.1:3000")
    repo.add("exp/t/gen_servers/1", "10.0.0.2:3000")
    with pytest.raises(name_resolve.NameEntryExistsError):
        repo.add("exp/t/gen_servers/0", "x")
    repo.add("exp/t/gen_servers/0", "10.0.0.9:1", replace=True)
    assert repo.get("exp/t/gen_servers/0") == "10.0.0.9:1"
    assert repo.get_subtree("exp/t/gen_servers") == ["10.0.0.9:1", "10.0.0.2:3000"]
    assert repo.find_subtree("exp/t/gen_servers") == ["exp/t/gen_servers/0", "exp/t/gen_servers/1"]
    sub = repo.add_subentry("exp/t/workers", "w")
    assert repo.get(sub) == "w"
    repo.delete("exp/t/gen_servers/1")
    with pytest.raises(name_resolve.NameEntryNotFoundError):
        repo.get("exp/t/gen_servers/1")
    with pytest.raises(TimeoutError):
        repo.wait("exp/t/none", timeout=0.1, poll_frequency=0.02)
    repo.clear_subtree("exp/t")
    assert repo.find_subtree("exp/t") == []
    with pytest.raises(ImportError):  # the etcd3 client library is not installed here
        name_resolve.make_repository(NameResolveConfig(type="etcd3"))
    with pytest.raises(ValueError):
        name_resolve.make_repository(NameResolveConfig(type="zookeeper"))


def test_seeding_is_deterministic_per_key():
    a = seeding.set_random_seed(1, "trainer0")
    x = torch.rand(3)
    b = seeding.set_random_seed(1, "trainer1")
    y = torch.rand(3)
    seeding.set_random_seed(1, "trainer0")
    assert a != b and not torch.equal(x, y) and torch.equal(torch.rand(3), x)
    assert seeding.get_shuffle_seed() == seeding.get_shuffle_seed()
