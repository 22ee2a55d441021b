"""Import shim: the package directory is named after the reference project and is not a Python identifier, so it
is loaded by path here and re-exported as ``fnx_b200``."""
import importlib.util
import pathlib
import sys

_DIR = pathlib.Path(__file__).resolve().parent / "qwen3.8-flash-next-2x-p100_b200"
_NAME = "qwen3_8_flash_next_2x_p100_b200"
if _NAME not in sys.modules:
    _spec = importlib.util.spec_from_file_location(_NAME, _DIR / "__init__.py", submodule_search_locations=[str(_DIR)])
    _mod = importlib.util.module_from_spec(_spec)
    sys.modules[_NAME] = _mod
    _spec.loader.exec_module(_mod)
_mod = sys.modules[_NAME]
globals().update({k: v for k, v in vars(_mod).items() if not k.startswith("__")})
PACKAGE_DIR = _DIR
