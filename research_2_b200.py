"""Import name for the package that lives in the folder `research-2_b200/`.

A hyphen cannot appear in a Python module name, so `import research_2_b200` finds this file,
which loads the folder's `__init__.py` as the package `research_2_b200` (its sub-packages
resolve through the folder's path as usual).
"""

import importlib.util
import pathlib
import sys

_folder = pathlib.Path(__file__).resolve().parent / "research-2_b200"
_spec = importlib.util.spec_from_file_location(
    "research_2_b200", _folder / "__init__.py", submodule_search_locations=[str(_folder)]
)
_module = importlib.util.module_from_spec(_spec)
sys.modules["research_2_b200"] = _module
_spec.loader.exec_module(_module)

if __name__ == "__main__":  # `python -m research_2_b200 ...` is the command line
    from research_2_b200.cli import main as _main

    sys.exit(_main())
