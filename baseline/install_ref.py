"""Install the unmodified reference package (xiaohuangji/MoC, `moc`) into baseline/_ref.

    python baseline/install_ref.py <path-to-reference-checkout>

baseline/_ref is not under version control; it travels with the working tree to machines that have no reference
checkout. It serves three purposes, all optional (everything falls back or skips when it is absent):
  * tests/test_dropin_gpu.py builds the reference's own LLaMAModel (moc/model.py) with the B200 FFN modules
    installed into it (moc_b200.install_into) - the real drop-in;
  * bench.py's CPU baseline and `--impl reference` arm time the reference's own MoCSwiGLUFFN(mode="moc")
    instead of the oracle restatement;
  * bench.py's `reference_gpu` record times the reference's stock CUDA path on the same GPU.

The source tree may be read-only, so the build runs on a temporary copy; dependency pins of the reference
(torch < 2.9, triton < 3.5) do not match this environment, hence --no-deps.
"""
from __future__ import annotations

import shutil
import subprocess
import sys
import tempfile
from pathlib import Path

TARGET = Path(__file__).resolve().parent / "_ref"


def install(reference_dir: str | Path, wheelhouse: str | None = None) -> Path:
    src = Path(reference_dir)
    if not (src / "moc" / "ffn.py").exists():
        raise FileNotFoundError(f"{src} is not a checkout of the reference (moc/ffn.py missing)")
    with tempfile.TemporaryDirectory() as tmp:
        work = Path(tmp) / "src"
        shutil.copytree(src, work, ignore=shutil.ignore_patterns(".git", "data", "results", "docs"))
        cmd = [sys.executable, "-m", "pip", "install", "--no-index", "--no-build-isolation", "--no-deps", "--upgrade",
               "--target", str(TARGET)]
        if wheelhouse:
            cmd += ["--find-links", wheelhouse]
        subprocess.run(cmd + [str(work)], check=True, capture_output=True, text=True)
    if not (TARGET / "moc" / "ffn.py").exists():
        raise RuntimeError("pip reported success but baseline/_ref/moc is missing")
    return TARGET


if __name__ == "__main__":
    if len(sys.argv) < 2:
        raise SystemExit(__doc__)
    print(install(sys.argv[1], sys.argv[2] if len(sys.argv) > 2 else None))
