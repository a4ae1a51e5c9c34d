"""Build/loader integrity on the CPU: content addressing, torch-free imports, doctor report."""

import json
import subprocess
import sys
from pathlib import Path

from afdep_b200 import _native

ROOT = Path(__file__).resolve().parents[1]


def test_digest_covers_every_native_source_and_changes_with_content(tmp_path, monkeypatch):
    files = _native.native_sources()
    names = {p.name for p in files}
    assert {"dispatch.cu", "ffn.cu", "combine.cu", "grouped_gemm.cu", "bindings.cpp", "ptx.cuh", "layout.h"} <= names
    before = _native.source_digest()
    # same names, one byte different in a header => different digest, even with an identical mtime
    clone = tmp_path / "csrc"
    for p in files:
        dst = clone / p.relative_to(_native.CSRC)
        dst.parent.mkdir(parents=True, exist_ok=True)
        dst.write_bytes(p.read_bytes())
    monkeypatch.setattr(_native, "CSRC", clone)
    assert _native.source_digest() == before
    header = clone / "include" / "afdep" / "layout.h"
    header.write_bytes(header.read_bytes() + b"\n// changed\n")
    assert _native.source_digest() != before
    assert _native.module_name().startswith("_afdep_native_") and len(_native.module_name()) == len("_afdep_native_") + 16


def test_package_and_loader_import_without_torch():
    code = (
        "import sys, afdep_b200, afdep_b200._native, afdep, afdep.deepep;"
        "bad=[m for m in ('torch','vllm','triton','deep_ep') if m in sys.modules];"
        "assert not bad, bad; print(afdep.Config(8,256,8,2,2,2).role_aware)"
    )
    out = subprocess.run([sys.executable, "-c", code], check=True, cwd=ROOT, capture_output=True, text=True)
    assert out.stdout.strip() == "True"


def test_doctor_reports_json_and_fails_without_a_gpu():
    for module in ("afdep_b200", "afdep"):
        proc = subprocess.run([sys.executable, "-m", module, "doctor"], cwd=ROOT, capture_output=True, text=True)
        report = json.loads(proc.stdout)
        assert report["source_digest"] == _native.source_digest()
        assert {"afdep_b200", "platform", "native_library", "errors", "nvcc"} <= set(report)
        import torch

        if not torch.cuda.is_available():
            assert proc.returncode == 1 and any("CUDA" in e for e in report["errors"])


def test_every_kernel_source_targets_sm100a_and_never_traps():
    assert "arch=compute_100a,code=sm_100a" in " ".join(_native.NVCC_FLAGS)
    for p in _native.native_sources():
        text = p.read_text()
        code = "\n".join(line.split("//")[0] for line in text.splitlines())
        assert "__trap" not in code and "asm(\"trap" not in code and "assert(" not in code.replace("static_assert(", ""), p.name


def test_build_signature_changes_with_the_toolchain(monkeypatch):
    base = _native.build_signature()
    assert base != _native.source_digest() and _native.module_name().endswith(base[:16])
    sig = dict(_native.toolchain_signature())
    assert {"torch", "python_abi", "nvcc", "arch"} <= set(sig)
    for key in ("torch", "python_abi", "nvcc"):
        changed = dict(sig, **{key: sig[key] + "-other"})
        monkeypatch.setattr(_native, "toolchain_signature", lambda changed=changed: changed)
        assert _native.build_signature() != base, key
