"""Allocation-mode mini-language: parsing, precedence, validation."""
import pytest

from areal_b200.api.alloc_mode import (AllocationMode, AllocationValidationError, InvalidAllocationModeError,
                                       ModelAllocation, ParallelStrategy, SchedulingStrategyType)

CASES = [
    ("sglang:d2+fsdp:d4", 2, "sglang", "fsdp", dict(gen_dp=2, train_dp=4)),
    ("native:d4+fsdp:d4", 2, "native", "fsdp", dict(gen_dp=4, train_dp=4)),
    ("sglang:d4p2t2+megatron:(attn:d2p2t2c2|ffn:d2p2t2e2)", 2, "sglang", "megatron", dict(train_cp=2, train_ep=2)),
    ("fsdp:d4", 1, None, "fsdp", dict(train_dp=4)),
    ("megatron:d2p2t1", 1, None, "megatron", dict(train_pp=2)),
    ("vllm:d2t4+megatron:d2p2t1", 2, "vllm", "megatron", dict(gen_tp=4)),
    ("archon:d2t2c2", 1, None, "archon", dict(train_cp=2, train_tp=2)),
    ("megatron:d2p2t2c2e4", 1, None, "megatron", dict(train_ep=4)),
    ("sglang[rollout]:d2+fsdp[actor]:d4+fsdp[critic]:d2", 3, "sglang", "fsdp", {}),
]


@pytest.mark.parametrize("expr,n,gen,train,dims", CASES)
def test_parsing(expr, n, gen, train, dims):
    m = AllocationMode.from_str(expr)
    assert len(m) == n
    assert m.gen_backend == gen and m.train_backend == train
    for k, v in dims.items():
        side, dim = k.split("_")
        strat = m.gen if side == "gen" else m.train
        assert getattr(strat, f"{dim}_size") == v


def test_world_sizes_and_properties():
    a = ModelAllocation.from_str("megatron:d2p2t2c2")
    assert a.world_size == 16 and a.parallel.world_size == 16
    p = ParallelStrategy(tensor_parallel_size=2, data_parallel_size=4, expert_parallel_size=4)
    assert p.expert_data_parallel_size == 2
    assert str(ParallelStrategy(data_parallel_size=2)) == "Parallel(tp=1,pp=1,dp=2)"
    assert ModelAllocation.from_str("sglang:d1").world_size == 1


def test_operator_precedence_and_colocation():
    m = AllocationMode.from_str("sglang[gen]:d4+fsdp[actor]:d4|fsdp[ref]:d4")
    assert [a.name for a in m.allocations] == ["gen", "actor", "ref"]
    assert m["ref"].scheduling_strategy.type == SchedulingStrategyType.colocation
    assert m["ref"].scheduling_strategy.target == "actor"
    assert m["actor"].scheduling_strategy.type == SchedulingStrategyType.separation
    assert m.world_size == 8


def test_hybrid_moe_derives_expert_dp():
    a = ModelAllocation.from_str("megatron:(attn:d1p12t4|ffn:d1p12e4)")
    assert a.parallel.ep_size == 4 and a.parallel.pp_size == 12 and a.parallel.tp_size == 4
    b = ModelAllocation.from_str("megatron:(attn:d4t2|ffn:e4)")
    assert b.parallel.world_size == 8 and b.parallel.expert_data_parallel_size == 2


@pytest.mark.parametrize("expr,exc", [
    ("fsdp:d2p2", AllocationValidationError),            # FSDP has no pipeline parallelism
    ("fsdp:d2e2", AllocationValidationError),
    ("d4", AllocationValidationError),                    # bare dims: backend required
    ("[actor]:d4", AllocationValidationError),
    ("(attn:d2|ffn:e2)", AllocationValidationError),
    ("fsdp[a]:d4|fsdp:d4", AllocationValidationError),    # colocated members need names
    ("fsdp[a]:d4|fsdp[b]:d2", AllocationValidationError), # and equal world sizes
    ("fsdp[a]:d2+fsdp[a]:d2", AllocationValidationError), # duplicate names
    ("sglang:d2+fsdp:d2+fsdp:d2", AllocationValidationError),  # 3+ components need names
    ("megatron:(attn:d2p2|ffn:p4e1)", AllocationValidationError),
    ("megatron:(attn:d4|ffn:d2e4)", InvalidAllocationModeError),
    ("sglang.d4", ValueError), ("fsdp:x4", ValueError), ("", ValueError), ("sglang:c2", ValueError),
])
def test_validation_errors(expr, exc):
    with pytest.raises(exc):
        AllocationMode.from_str(expr)


def test_from_str_rejects_multi_component():
    with pytest.raises(AllocationValidationError):
        ModelAllocation.from_str("sglang:d2+fsdp:d2")
    a = ModelAllocation.from_str("fsdp:d4", name="actor")
    assert a.name == "actor"
