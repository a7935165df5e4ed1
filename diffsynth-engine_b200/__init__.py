"""B200 (sm_100a) kernels for the DiT denoising step of DiffSynth-Engine, behind the engine's own
seams: the attention-function dispatch, the patched ``F.linear`` quantised-Linear API and the
multi-GPU model wrapper.  Everything computes in ``libdsb.so`` (see ``include/dsb.h``)."""
from . import _lib, ops  # noqa: F401
from ._lib import DsbError  # noqa: F401

__version__ = "0.1.0"
