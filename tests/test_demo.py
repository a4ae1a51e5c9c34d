"""The demo program (`python -m afdep_b200.models.demo`) as ranks of a job: on CPU over the Gloo
transport with torch experts here, on real GPUs with the tcgen05 experts in the GPU run."""

import pytest

from tests._dist import run_ranks


def _demo(rank, world, backend):
    from afdep_b200.models import demo

    result = demo.main(["--ffn", str(world // 2), "--backend", backend, "--tokens", "48", "--steps", "2"])
    assert result["ok"] and result["ranks"] == world and result["max_relative_error"] < 3e-2


def test_demo_layer_on_four_cpu_ranks():
    run_ranks(_demo, 4, "gloo", timeout=300)


@pytest.mark.gpu
@pytest.mark.multigpu(2)
def test_demo_layer_on_two_gpus():
    run_ranks(_demo, 2, "native", timeout=600)
