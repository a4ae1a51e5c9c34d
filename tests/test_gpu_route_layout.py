"""The stand-alone routing-layout kernel against its plain-torch statement."""

import pytest
import torch

from afdep_b200.ops.route_layout import reference_layout, route_layout
from afdep_b200.utils import synthetic

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("tokens,experts,ffn,top_k", [(0, 8, 2, 2), (1, 8, 1, 2), (37, 16, 2, 4), (300, 64, 4, 8), (2048, 256, 4, 8), (513, 60, 3, 5), (129, 256, 8, 32)])
def test_layout_matches_reference(tokens, experts, ffn, top_k):
    gen = torch.Generator().manual_seed(tokens + experts)
    ids = synthetic.distinct_routes(tokens, experts, top_k, gen)
    if tokens:
        drop = torch.rand(ids.shape, generator=gen) < 0.15
        ids = torch.where(drop, torch.full_like(ids, -1), ids)
    if tokens > 10:
        ids[5, 0] = experts + 3          # an illegal token publishes nothing
        ids[7, 1] = ids[7, 0] if ids[7, 0] >= 0 else ids[7, 1]
    got = [t.cpu() for t in route_layout(ids.cuda(), experts, ffn)]
    want = reference_layout(ids, experts, ffn)
    for name, g, w in zip(("route_e", "route_pos", "tok_slot", "counts"), got, want):
        assert torch.equal(g, w), name
