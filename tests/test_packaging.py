"""Install the package into a scratch directory with pip (offline, no build isolation) and import it with an
interpreter that sees nothing else (`python -I -S`): the control plane must work without torch, and the
missing native pieces must be reported, not crash.  Mirrors the reference's packaging tier
(tests/packaging/test_install_matrix.py:10-72)."""

import os
import shutil
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.timeout(600)
def test_pip_install_and_torch_free_import(tmp_path):
    # install from a copy: pip writes build/ and *.egg-info next to the sources
    source = tmp_path / "src"
    source.mkdir()
    for name in ("pyproject.toml", "setup.py", "README.md"):
        shutil.copy(os.path.join(ROOT, name), source / name)
    shutil.copytree(os.path.join(ROOT, "lowbit_comm_b200"), source / "lowbit_comm_b200",
                    ignore=shutil.ignore_patterns("*.so", "*.o", "build", "__pycache__"))
    target = tmp_path / "site"
    env = dict(os.environ, LBC_BUILD_NATIVE="")
    proc = subprocess.run([sys.executable, "-m", "pip", "install", "--no-index", "--no-build-isolation", "--no-deps",
                           "--quiet", "--target", str(target), str(source)], env=env, capture_output=True, text=True,
                          timeout=500)
    assert proc.returncode == 0, proc.stdout[-2000:] + proc.stderr[-2000:]
    pkg = target / "lowbit_comm_b200"
    assert (pkg / "core" / "plan.py").exists() and (pkg / "ops" / "csrc" / "fast_kernels.cu").exists()
    assert (pkg / "ops" / "csrc" / "host_codec.cpp").exists()
    code = (
        "import sys; sys.path.insert(0, %r)\n"
        "import lowbit_comm_b200 as lbc\n"
        "assert 'torch' not in sys.modules, 'the package imported torch'\n"
        "cfg = lbc.CompressionConfig(bit=8, group_size=64)\n"
        "plan = lbc.CommunicationPlan(collective='all_reduce', strategy='auto', compression=cfg)\n"
        "ctx = lbc.CompileContext(rank=0, world_size=2, device='cuda:0', shape=(1024,), dtype='bf16')\n"
        "decision = lbc.CCDLCommunicationPlugin().plan({'training_backend': 'native_ddp', 'device_type': 'cuda'}, cfg)\n"
        "report = lbc.detect()\n"
        "assert report.available is False and report.reason, report\n"
        "assert 'torch' not in sys.modules\n"
        "print('OK', decision.enabled, plan.strategy, ctx.world_size, lbc.__version__)\n"
    ) % str(target)
    run = subprocess.run([sys.executable, "-I", "-S", "-c", code], capture_output=True, text=True, timeout=120)
    assert run.returncode == 0, run.stdout + run.stderr
    assert run.stdout.strip().startswith("OK")
