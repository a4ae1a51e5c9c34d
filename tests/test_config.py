"""Config contract: geometry, receive bounds and validation messages (CPU, no torch)."""

import subprocess
import sys
from dataclasses import replace

import pytest

from afdep_b200 import Config


def cfg(**kw):
    base = dict(capacity_tokens_per_rank=16, hidden_size=256, num_experts=16, top_k=16, ffn_ranks=2, attention_ranks=2, role_aware=False)
    return Config(**(base | kw))


def test_expert_geometry():
    c = cfg()
    assert (c.world_size, c.experts_per_rank, c.logical_experts) == (4, 8, 32)
    assert c.top_k > c.experts_per_rank
    with pytest.raises(ValueError, match="divide evenly"):
        cfg(num_experts=15)


def test_receive_bound_counts_only_sources_when_role_aware():
    generic = cfg(capacity_tokens_per_rank=2048)
    roles = replace(generic, role_aware=True)
    assert generic.receive_rows(2048) == 66_560
    assert roles.receive_rows(2048) == 33_792
    assert roles.logical_experts == generic.logical_experts


def test_default_comm_sm_share_on_b200():
    assert cfg().resolved_num_sms(148) == 27
    assert cfg(num_sms=12).resolved_num_sms(148) == 12
    assert cfg().resolved_num_sms(8) == 4


@pytest.mark.parametrize(
    "kwargs, message",
    [
        ({"capacity_tokens_per_rank": 0}, "positive int32"),
        ({"hidden_size": True}, "positive int32"),
        ({"num_sms": -1}, "nonnegative int32"),
        ({"num_qps": 1 << 31}, "nonnegative int32"),
        ({"hidden_size": 384}, "multiple of 256"),
        ({"num_experts": 31, "top_k": 2}, "divide evenly"),
        ({"top_k": 33, "num_experts": 64}, "top_k"),
        ({"allow_hybrid_mode": 1}, "boolean"),
        ({"role_aware": 1}, "role_aware must be a boolean"),
        ({"payload": "fp16"}, "payload"),
        ({"rdma_traffic_class": 256}, "traffic_class"),
        ({"capacity_tokens_per_rank": (1 << 31) - 2, "top_k": 16}, "int32 indexing"),
        ({"ffn_ranks": 1, "num_experts": 512, "top_k": 8}, "workspace bounds"),
    ],
)
def test_invalid_configs(kwargs, message):
    with pytest.raises(ValueError, match=message):
        cfg(**kwargs)


def test_public_import_needs_no_torch():
    code = (
        "import sys, afdep_b200, afdep_b200._native;"
        "from afdep_b200 import Buffer, Config, ReceiveResult;"
        "assert Config(8,256,8,2,2,2).role_aware;"
        "bad=[m for m in ('torch','vllm','triton') if m in sys.modules];"
        "assert not bad, bad"
    )
    subprocess.run([sys.executable, "-c", code], check=True, cwd=str(__import__('pathlib').Path(__file__).resolve().parents[1]))
