"""Puts the unmodified reference under baseline/_ref, for bench.py's reference arm.

    python baseline/install_reference.py [SOURCE_TREE]

First the packaged route, `pip install --no-index --no-build-isolation --find-links
/opt/wheelhouse --target baseline/_ref SOURCE_TREE`; the reference's build backend
(hatchling, pyproject.toml:44-46) is not in the offline wheelhouse, so this fails there and
the outcome is recorded in baseline/_ref/INSTALL.json.  Then the plain route, which is all
an install of a pure-Python package is: a copy of the reference's `model` package (and its
pyproject.toml), nothing edited, and its paged-attention extension built in place with its
own setup.py and its own documented switch for another GPU (model/kernels/setup.py:8-9,20:
"set TORCH_CUDA_ARCH_LIST to build for something else").  nvcc cross-compiles without a GPU.
"""

import json
import os
import shutil
import subprocess
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
DEST = HERE / "_ref"


def installed():
    return (DEST / "model" / "inference_paged.py").exists()


def extension_built():
    return any((DEST / "model" / "kernels").glob("_C*.so"))


def install(source, log=print):
    source = Path(source)
    if not (source / "model" / "inference_paged.py").exists():
        log(f"install_reference: no reference source tree at {source}")
        return False
    record = {"source": str(source)}
    if not installed():
        DEST.mkdir(parents=True, exist_ok=True)
        pip = subprocess.run(
            [sys.executable, "-m", "pip", "install", "--no-index", "--no-build-isolation", "--find-links",
             "/opt/wheelhouse", "--no-deps", "--target", str(DEST), str(source)],
            capture_output=True, text=True)
        record["pip_returncode"] = pip.returncode
        record["pip_error"] = (pip.stderr or pip.stdout).strip().splitlines()[-1:] if pip.returncode else []
        if not installed():
            shutil.copytree(source / "model", DEST / "model")
            shutil.copy(source / "pyproject.toml", DEST / "pyproject.toml")
            for p in DEST.rglob("*"):                     # the source tree may be read-only
                p.chmod(p.stat().st_mode | 0o200)
            record["route"] = "plain copy of the model package"
        else:
            record["route"] = "pip"
    if not extension_built():
        env = dict(os.environ, TORCH_CUDA_ARCH_LIST="10.0")
        build = subprocess.run([sys.executable, "setup.py", "build_ext", "--inplace"],
                               cwd=DEST / "model" / "kernels", env=env, capture_output=True, text=True)
        record["extension_returncode"] = build.returncode
        if build.returncode:
            record["extension_error"] = build.stderr.strip().splitlines()[-5:]
    record["extension_built"] = extension_built()
    (DEST / "INSTALL.json").write_text(json.dumps(record, indent=1))
    log(f"install_reference: {json.dumps(record)}")
    return installed()


if __name__ == "__main__":
    src = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("SOCRATES_REFERENCE_SRC", "/root/reference")
    sys.exit(0 if install(src) else 1)
