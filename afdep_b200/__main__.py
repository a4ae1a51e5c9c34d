"""``python -m afdep_b200 doctor [--build]``: report what the library needs and what it finds.

Prints one JSON document and exits 1 if ``errors`` is non-empty.  Nothing here creates a
Buffer, talks to another rank or changes a device setting.  Same role as the reference's
``python -m afdep doctor`` (afdep/__main__.py:14-69), with the NCCL probes replaced by the
things this transport depends on: CUDA virtual-memory export and peer access over NVLink.
"""

from __future__ import annotations

import argparse
import json
import platform

from . import __version__
from ._native import build_signature, library_path, load_native, resolve_nvcc, source_digest, stale_libraries, toolchain_signature


def report(build: bool) -> dict:
    out: dict = {
        "afdep_b200": __version__,
        "platform": platform.platform(),
        "source_digest": source_digest(),
        "build_signature": build_signature(),
        "toolchain": toolchain_signature(),
        "native_library": str(library_path()),
        "native_library_built": library_path().exists(),
        "stale_libraries": [p.name for p in stale_libraries()],
        "errors": [],
    }
    try:
        out["nvcc"] = resolve_nvcc()
    except RuntimeError as exc:
        out["errors"].append(str(exc))
    try:
        import torch

        out.update(torch=torch.__version__, torch_cuda=torch.version.cuda, cuda_available=torch.cuda.is_available())
        if torch.cuda.is_available():
            count = torch.cuda.device_count()
            props = torch.cuda.get_device_properties(torch.cuda.current_device())
            out.update(
                gpu=props.name,
                capability=list(torch.cuda.get_device_capability()),
                sm_count=props.multi_processor_count,
                device_count=count,
                memory_gib=round(props.total_memory / 2**30, 1),
            )
            if tuple(out["capability"]) != (10, 0):
                out["errors"].append("kernels are built for sm_100a only; this device is not a B200-class GPU")
            peers = {}
            for i in range(count):
                peers[str(i)] = [j for j in range(count) if j != i and torch.cuda.can_device_access_peer(i, j)]
            out["peer_access"] = peers
            if count > 1 and any(len(v) != count - 1 for v in peers.values()):
                out["errors"].append("not every GPU pair has peer access; the symmetric heap needs one NVLink domain")
        else:
            out["errors"].append("No CUDA GPU is available")
    except ImportError as exc:
        out["errors"].append(str(exc))
    if build:
        try:
            module = load_native()
            out["native_library_built"] = True
            out["native_module"] = module.__name__
            out["native_max_ranks"] = int(module.max_ranks)
            out["native_build"] = dict(module.build_info())
            import torch

            if torch.cuda.is_available():
                vmm = bool(module.vmm_supported(torch.cuda.current_device()))
                out["heap_mode"] = "vmm (POSIX file descriptors)" if vmm else "cudaIpc"
        except Exception as exc:  # noqa: BLE001 - the report is the product
            out["errors"].append(f"{type(exc).__name__}: {exc}")
    return out


def main(argv: list[str] | None = None) -> None:
    parser = argparse.ArgumentParser(prog="afdep_b200", description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    parser.add_argument("command", choices=["doctor"])
    parser.add_argument("--build", action="store_true", help="compile (if needed) and load the CUDA extension")
    args = parser.parse_args(argv)
    out = report(args.build)
    print(json.dumps(out, indent=2))
    if out["errors"]:
        raise SystemExit(1)


if __name__ == "__main__":
    main()
