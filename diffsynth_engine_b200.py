"""Import alias.  The package lives in the directory ``diffsynth-engine_b200`` (with a hyphen, which Python cannot
import by name); importing ``diffsynth_engine_b200`` with the repository root on ``sys.path`` loads that directory
as this module.  Worker processes started with ``multiprocessing`` rely on it to unpickle their entry point."""
import importlib.util
import os
import sys

_dir = os.path.join(os.path.dirname(os.path.abspath(__file__)), "diffsynth-engine_b200")
_spec = importlib.util.spec_from_file_location(__name__, os.path.join(_dir, "__init__.py"),
                                               submodule_search_locations=[_dir])
_mod = importlib.util.module_from_spec(_spec)
sys.modules[__name__] = _mod
_spec.loader.exec_module(_mod)
