"""Installs the UNMODIFIED reference (modelscope/DiffSynth-Engine) into ``baseline/_ref`` with pip, offline:

    python baseline/install_reference.py [path to the DiffSynth-Engine source tree]

``baseline/_ref`` is not version-controlled; it is only used by the GPU drop-in tests
(``tests/test_reference_dropin_gpu.py``, skipped when it is absent) and by ``bench.py --workload reference-gpu``,
which drive the reference's own modules.  ``--no-deps``: the hot-path modules need torch, einops and safetensors,
which are present; the package's download / video helpers need modules that are not, so the tests import the
hot-path modules through a bare namespace package (see ``import_reference`` below)."""
import os
import subprocess
import sys
import types

HERE = os.path.dirname(os.path.abspath(__file__))
TARGET = os.path.join(HERE, "_ref")
# default place of the reference's source tree: a directory ``reference`` beside this repository
DEFAULT_SOURCE = os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference")


def install(source: str = DEFAULT_SOURCE, force: bool = False) -> bool:
    """True when ``baseline/_ref`` holds the package afterwards."""
    if os.path.isdir(os.path.join(TARGET, "diffsynth_engine")) and not force:
        return True
    if not os.path.isdir(source):
        return False
    cmd = [sys.executable, "-m", "pip", "install", "--no-index", "--no-build-isolation", "--no-deps",
           "--find-links", "/opt/wheelhouse", "--target", TARGET, "--upgrade", source]
    r = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if r.returncode != 0:
        sys.stderr.write(r.stdout[-2000:])
        return False
    return os.path.isdir(os.path.join(TARGET, "diffsynth_engine"))


def import_reference():
    """The reference's hot-path modules from ``baseline/_ref`` (None when it is not installed).  The package's
    ``__init__`` pulls in download and video helpers whose dependencies are absent, so a bare namespace package is
    registered in its place and the sub-modules are imported directly."""
    pkg_dir = os.path.join(TARGET, "diffsynth_engine")
    if not os.path.isdir(pkg_dir):
        return None
    if "diffsynth_engine" not in sys.modules:
        m = types.ModuleType("diffsynth_engine")
        m.__path__ = [pkg_dir]
        sys.modules["diffsynth_engine"] = m
    from diffsynth_engine.models.basic import transformer_helper
    from diffsynth_engine.models.flux import flux_dit
    from diffsynth_engine.models.wan import wan_dit
    from diffsynth_engine.utils import fp8_linear
    return types.SimpleNamespace(flux_dit=flux_dit, wan_dit=wan_dit, transformer_helper=transformer_helper,
                                 fp8_linear=fp8_linear)


if __name__ == "__main__":
    ok = install(*([a for a in sys.argv[1:] if not a.startswith("--")][:1] or [DEFAULT_SOURCE]), force="--force" in sys.argv)
    print("installed" if ok else "not installed")
