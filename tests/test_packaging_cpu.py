"""The package installs with pip and registers the `torch.backends` entry point, so that a plain
`import torch` loads the spyre backend (pyproject.toml:62-63 and torch_spyre/__init__.py:140-163 of
the reference)."""
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_pip_install_and_autoload(tmp_path):
    # install from a copy: pip builds in the source directory and would leave an egg-info there, whose
    # entry point any later `import torch` with that directory on sys.path would pick up
    import shutil
    src = tmp_path / "src"
    shutil.copytree(os.path.join(ROOT, "torch-spyre_b200"), src,
                    ignore=shutil.ignore_patterns("build", "*.egg-info", "__pycache__"))
    shutil.copytree(os.path.join(ROOT, "include"), tmp_path / "include")     # build.py looks for ../include
    target = tmp_path / "site"
    out = subprocess.run([sys.executable, "-m", "pip", "install", "--no-deps", "--no-build-isolation", "--no-index",
                          "--quiet", "--target", str(target), str(src)],
                         capture_output=True, text=True, timeout=900)
    assert out.returncode == 0, out.stderr[-2000:]
    eps = (target / "torch_spyre-0.2.0.dist-info" / "entry_points.txt").read_text()
    assert "[torch.backends]" in eps and "torch_spyre = torch_spyre:_autoload" in eps
    assert (target / "torch_spyre" / "lib" / "libspyre_b200.so").exists() and (target / "torch_spyre" / "_C.so").exists()
    env = {k: v for k, v in os.environ.items() if k != "PYTHONPATH"}
    env["PYTHONPATH"] = str(target)
    code = ("import torch, sys; assert 'torch_spyre' in sys.modules, 'not autoloaded'; "
            "print(torch._C._get_privateuse1_backend_name(), hasattr(torch, 'spyre'), "
            "sys.modules['torch_spyre'].__file__)")
    run = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, cwd=str(tmp_path), env=env,
                         timeout=600)
    assert run.returncode == 0, run.stderr[-2000:]
    name, has_module, where = run.stdout.split()
    assert name == "spyre" and has_module == "True" and where.startswith(str(target))
    # and autoload can be switched off the way torch documents it
    env["TORCH_DEVICE_BACKEND_AUTOLOAD"] = "0"
    off = subprocess.run([sys.executable, "-c", "import torch, sys; print('torch_spyre' in sys.modules)"],
                         capture_output=True, text=True, cwd=str(tmp_path), env=env, timeout=600)
    assert off.returncode == 0 and off.stdout.strip() == "False"
