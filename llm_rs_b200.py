"""Import shim: makes the package folder ``llm-rs_b200/`` importable as ``llm_rs_b200``.

The package folder carries the project's name, which holds a hyphen and so cannot be
written in an ``import`` statement. ``import llm_rs_b200`` finds this file; it loads
the folder's ``__init__.py`` as the real package (with its sub-packages) and puts
that in ``sys.modules`` under the importable name. Run as ``python -m llm_rs_b200 ...`` it is the command line.
"""
import importlib.util
import os
import sys

_pkg_dir = os.path.join(os.path.dirname(os.path.abspath(__file__)), "llm-rs_b200")
_spec = importlib.util.spec_from_file_location(
    "llm_rs_b200", os.path.join(_pkg_dir, "__init__.py"),
    submodule_search_locations=[_pkg_dir])
_module = importlib.util.module_from_spec(_spec)
sys.modules["llm_rs_b200"] = _module
_spec.loader.exec_module(_module)

if __name__ == "__main__":      # ``python -m llm_rs_b200 <command> ...`` runs this file: hand over to the command line
    from llm_rs_b200.cli import main
    sys.exit(main())
