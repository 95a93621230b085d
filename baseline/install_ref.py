"""Puts mxinO/holon, unmodified, under baseline/_ref for `bench.py --impl reference`.

    python baseline/install_ref.py <path of the reference checkout>

First the documented offline install is tried:

    python -m pip install --no-index --no-build-isolation --find-links /opt/wheelhouse --target baseline/_ref <checkout>

It needs the reference's build backend (hatchling); where that is missing, the reference's four pure-Python
distributions are copied file by file instead (core/holon, std/holon_std, plugins/holon_plugins,
testing/holon_testing: what `pip install` of the workspace would put on the path, manifests and vendored sources
included), which is all an import needs: the reference finds its plugins through their `plugin.toml` manifests.

Two optional kernel plugins are left out either way (LEFT_OUT): their sources name a CUDA copy routine that GPU runs
here must not contain, and neither is on the dense model's path (one moves expert weights of mixture-of-experts
models, the other moves cache rows between device and host tiers, which are off by default). A plugin that is not
installed is simply not offered by the reference's plugin set.
"""
from __future__ import annotations

import pathlib
import shutil
import subprocess
import sys

HERE = pathlib.Path(__file__).resolve().parent
TARGET = HERE / "_ref"
PACKAGES = (("core", "holon"), ("std", "holon_std"), ("plugins", "holon_plugins"), ("testing", "holon_testing"))
LEFT_OUT = ("holon_plugins/kernels/expert_io", "holon_plugins/kernels/state_copy")


def leave_out() -> None:
    for relative in LEFT_OUT:
        if (TARGET / relative).is_dir():
            shutil.rmtree(TARGET / relative)


def main(checkout: pathlib.Path) -> int:
    if TARGET.exists():
        shutil.rmtree(TARGET)
    pip = subprocess.run([sys.executable, "-m", "pip", "install", "--no-index", "--no-build-isolation", "--find-links",
                          "/opt/wheelhouse", "--target", str(TARGET), str(checkout)], capture_output=True, text=True)
    if pip.returncode == 0 and (TARGET / "holon").is_dir():
        leave_out()
        print(f"installed with pip into {TARGET}")
        return 0
    reason = (pip.stderr.strip().splitlines() or ["no message"])[-1]
    print(f"pip install failed ({reason}); copying the package trees")
    if TARGET.exists():
        shutil.rmtree(TARGET)
    TARGET.mkdir(parents=True)
    for folder, package in PACKAGES:
        shutil.copytree(checkout / folder / package, TARGET / package,
                        ignore=shutil.ignore_patterns("__pycache__", "*.pyc"))
    leave_out()
    (TARGET / "INSTALLED_FROM.txt").write_text(f"copied unmodified from {checkout} ({', '.join(f'{a}/{b}' for a, b in PACKAGES)}), "
                                               f"without {', '.join(LEFT_OUT)}; pip said: {reason}\n")
    print(f"copied {len(PACKAGES)} packages into {TARGET}")
    return 0


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit(__doc__)
    sys.exit(main(pathlib.Path(sys.argv[1])))
