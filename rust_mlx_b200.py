"""Import shim: the package lives in the folder ``rust-mlx_b200`` (a name Python
cannot import directly); ``import rust_mlx_b200`` loads that folder as a package."""
import importlib.util
import os
import sys

_dir = os.path.join(os.path.dirname(os.path.abspath(__file__)), "rust-mlx_b200")
_spec = importlib.util.spec_from_file_location(
    "rust_mlx_b200", os.path.join(_dir, "__init__.py"), submodule_search_locations=[_dir]
)
_module = importlib.util.module_from_spec(_spec)
sys.modules["rust_mlx_b200"] = _module
_spec.loader.exec_module(_module)
