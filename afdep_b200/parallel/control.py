"""CPU control plane of a Buffer: object all-gather and barrier among the ranks.

The data plane never goes through here.  The control plane runs at construction (agreeing on
settings, passing heap handles around), at ``close()`` and nowhere else, exactly the role
the caller-owned Gloo group plays in the reference (afdep/deepep.py:285-316, 514-529).
"""

from __future__ import annotations


class GlooControl:
    """Control plane over a caller-owned ``torch.distributed`` CPU (Gloo) group."""

    def __init__(self, group) -> None:
        import torch.distributed as dist

        self._dist, self._group = dist, group
        self.rank, self.size = group.rank(), group.size()

    def all_gather(self, value) -> list:
        values = [None] * self.size
        self._dist.all_gather_object(values, value, group=self._group)
        return values

    def barrier(self) -> None:
        self._dist.barrier(group=self._group)

    def check_backend(self, backend: str) -> None:
        dist = self._dist
        if not dist.is_initialized() or str(dist.get_backend(self._group)) != "gloo":
            raise ValueError("afdep bootstrap requires an initialized CPU Gloo group")

    def local_probe(self, backend: str) -> dict:
        return probe_device(backend)


class LocalControl:
    """Control plane of a loopback world: all ranks live in this process and agree trivially."""

    def __init__(self, rank: int, size: int) -> None:
        self.rank, self.size = rank, size

    def all_gather(self, value) -> list:
        return [value] * self.size

    def barrier(self) -> None:
        return None

    def check_backend(self, backend: str) -> None:
        if backend != "native":
            raise ValueError("a loopback world only runs the native transport")

    def local_probe(self, backend: str) -> dict:
        return probe_device(backend)


def probe_device(backend: str) -> dict:
    """What construction needs to know about this rank's device, or an exception."""
    if backend == "gloo":
        return {"sms": 0, "device": None, "source": ""}
    import torch

    if not torch.cuda.is_available() or torch.cuda.is_current_stream_capturing():
        raise RuntimeError("Create afdep buffers on CUDA, outside graph capture")
    device = torch.cuda.current_device()
    sms = torch.cuda.get_device_properties(device).multi_processor_count
    source = ""
    if backend == "native":
        from .._native import load_native, source_digest

        load_native()
        source = source_digest()
    return {"sms": sms, "device": device, "source": source}


def make_control(group):
    if isinstance(group, (GlooControl, LocalControl)):
        return group
    return GlooControl(group)
