"""The install metadata: the hyphenated source folder installs as the package ``llm_pipeline_b200`` with its CUDA
sources, and the console script of ``pyproject.toml`` runs (the reference ships ``llm-pipeline =
"llm_pipeline.cli:main"``, pyproject.toml:90-91 there)."""

import os
import shutil
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_every_subpackage_is_listed():
    import tomllib
    with open(os.path.join(ROOT, "pyproject.toml"), "rb") as f:
        meta = tomllib.load(f)
    listed = set(meta["tool"]["setuptools"]["packages"])
    source = os.path.join(ROOT, meta["tool"]["setuptools"]["package-dir"]["llm_pipeline_b200"])
    found = {"llm_pipeline_b200"}
    for name in sorted(os.listdir(source)):
        folder = os.path.join(source, name)
        if os.path.isdir(folder) and (os.path.isfile(os.path.join(folder, "__init__.py")) or name == "csrc"):
            found.add(f"llm_pipeline_b200.{name}")
    assert listed == found
    assert meta["project"]["scripts"]["llm-pipeline-b200"] == "llm_pipeline_b200.cli:main"


def test_installs_offline_and_the_console_script_runs(tmp_path):
    source = tmp_path / "source"
    source.mkdir()
    for name in ("pyproject.toml", "README.md"):
        shutil.copy(os.path.join(ROOT, name), source / name)
    shutil.copytree(os.path.join(ROOT, "llm-pipeline_b200"), source / "llm-pipeline_b200",
                    ignore=shutil.ignore_patterns("_build", "__pycache__"))
    target = tmp_path / "site"
    proc = subprocess.run([sys.executable, "-m", "pip", "install", "--no-index", "--no-build-isolation", "--no-deps", "--quiet",
                           "--target", str(target), str(source)], capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stdout[-2000:] + proc.stderr[-2000:]
    assert (target / "llm_pipeline_b200" / "csrc" / "gemm_stream.cu").is_file()
    assert (target / "llm_pipeline_b200" / "csrc" / "tcgen05.cuh").is_file()
    env = dict(os.environ, PYTHONPATH=str(target))
    proc = subprocess.run([sys.executable, str(target / "bin" / "llm-pipeline-b200"), "--help"], capture_output=True, text=True,
                          timeout=300, env=env, cwd=str(tmp_path))
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert "infer" in proc.stdout and "random-model" in proc.stdout and "replay" in proc.stdout
    where = subprocess.run([sys.executable, "-c", "import llm_pipeline_b200.engine as e; print(e.__file__)"], capture_output=True,
                           text=True, timeout=300, env=env, cwd=str(tmp_path))
    assert where.returncode == 0 and str(target) in where.stdout, where.stdout + where.stderr
