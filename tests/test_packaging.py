"""The wheel must carry everything a user needs to build the sm_100a library on their own box:
every native source, the type marker and the licence; and the installed copy must hash to the
same source digest as the tree it was built from.

The reference checks its distributions the same way (tests/check_distribution.py:1-54 and the
import check of .github/workflows/ci.yml:21-33).  The wheel is built offline from a scratch
copy, so the working tree is left untouched.
"""

import shutil
import subprocess
import sys
import zipfile
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]


@pytest.fixture(scope="module")
def wheel(tmp_path_factory):
    src = tmp_path_factory.mktemp("src")
    ignore = shutil.ignore_patterns("_lib", "__pycache__", "*.so", "*.o")
    for name in ("afdep_b200", "afdep"):
        shutil.copytree(ROOT / name, src / name, ignore=ignore)
    for name in ("pyproject.toml", "README.md", "LICENSE", "MANIFEST.in"):
        shutil.copy(ROOT / name, src / name)
    out = tmp_path_factory.mktemp("dist")
    cmd = [sys.executable, "-m", "pip", "wheel", str(src), "--no-deps", "--no-build-isolation", "--no-index", "-q", "-w", str(out)]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        pytest.skip("offline wheel build unavailable: " + proc.stderr[-300:])
    wheels = list(out.glob("afdep_b200-*.whl"))
    assert len(wheels) == 1
    return wheels[0]


def test_wheel_ships_every_native_source_and_the_licence(wheel):
    from afdep_b200 import _native

    names = set(zipfile.ZipFile(wheel).namelist())
    for path in _native.native_sources():
        assert str(path.relative_to(ROOT)) in names, f"{path.name} missing from the wheel"
    assert "afdep_b200/py.typed" in names
    assert "afdep/__init__.py" in names and "afdep/__main__.py" in names
    assert any(n.endswith("LICENSE") for n in names)
    assert not any(n.endswith(".so") for n in names), "the wheel is source-only; the library is built on the target box"


def test_installed_wheel_imports_without_torch_and_has_the_same_digest(wheel, tmp_path):
    from afdep_b200 import _native

    target = tmp_path / "site"
    subprocess.run([sys.executable, "-m", "pip", "install", str(wheel), "--no-deps", "--no-index", "-q", "--target", str(target)], check=True)
    code = (
        "import sys\n"
        "sys.modules['torch'] = None\n"             # any `import torch` now raises ImportError
        f"sys.path.insert(0, {str(target)!r})\n"
        "import afdep_b200, afdep\n"
        "from afdep_b200 import _native\n"
        f"assert afdep_b200.__file__.startswith({str(target)!r}), afdep_b200.__file__\n"
        "assert afdep_b200.Config(8, 256, 8, 2, 2, 2).role_aware\n"
        "assert afdep.Config is afdep_b200.Config\n"
        "print(_native.source_digest())\n"
    )
    proc = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, cwd=tmp_path)
    assert proc.returncode == 0, proc.stderr
    assert proc.stdout.strip() == _native.source_digest()
