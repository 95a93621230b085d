"""The compiler front of the kernels: a part's own CUDA files become a library of their own, named by what it was
made from. (Cross-compiling for sm_100a needs nvcc, no GPU.)"""
from __future__ import annotations

import pathlib
import shutil

import pytest

from holon_b200.kernels.build import BuildError, extension_path, nvcc_path

TOY = pathlib.Path(__file__).resolve().parent / "toy_kernels" / "toy_gate.cu"


def have_nvcc() -> bool:
    try:
        nvcc_path()
        return True
    except BuildError:
        return False


def test_an_extension_needs_a_name_and_files(tmp_path):
    with pytest.raises(BuildError, match="identifier"):
        extension_path("toy gate", [TOY], build_dir=tmp_path)
    with pytest.raises(BuildError, match="no such file"):
        extension_path("toy", [tmp_path / "missing.cu"], build_dir=tmp_path)
    with pytest.raises(BuildError, match="no sources"):
        extension_path("toy", [], build_dir=tmp_path)


@pytest.mark.skipif(not have_nvcc(), reason="nvcc is not installed")
def test_an_extension_is_compiled_once_and_again_when_its_source_changes(tmp_path, capsys):
    source = tmp_path / "src" / "toy_gate.cu"
    source.parent.mkdir()
    shutil.copy(TOY, source)
    first = extension_path("toy", [source], verbose=True)
    assert first.parent == source.parent / "_build" and first.name.startswith("libholon_b200x_toy_")
    assert "compiling 1 CUDA files" in capsys.readouterr().err
    assert extension_path("toy", [source], verbose=True) == first
    assert "compiling" not in capsys.readouterr().err                      # found, not built again
    source.write_text(source.read_text() + "\n// changed\n")
    second = extension_path("toy", [source], verbose=False)
    assert second != first and second.is_file() and not first.exists()    # the library of the earlier source is gone
    broken = tmp_path / "broken.cu"
    broken.write_text("this is no CUDA\n")
    with pytest.raises(BuildError, match="nvcc failed on broken.cu"):
        extension_path("broken", [broken], build_dir=tmp_path / "out", verbose=False)
