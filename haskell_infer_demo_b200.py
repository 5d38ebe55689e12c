"""Import shim: the package directory is named after the reference project and carries a hyphen
(`haskell-infer-demo_b200/`), which Python cannot import by name.  `import
haskell_infer_demo_b200` loads that directory as a regular package under this module's name."""
import importlib.util
import os
import sys

_dir = os.path.join(os.path.dirname(os.path.abspath(__file__)), "haskell-infer-demo_b200")
_spec = importlib.util.spec_from_file_location(
    __name__, os.path.join(_dir, "__init__.py"), submodule_search_locations=[_dir])
_module = importlib.util.module_from_spec(_spec)
sys.modules[__name__] = _module
_spec.loader.exec_module(_module)
